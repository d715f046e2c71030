* c5315 (c5315: 9-bit ALU): 137 gates, 1054 transistors
VDD vdd 0 DC 1.8
VIN0 na0 0 PULSE(0 1.8 5e-10 20p 20p 1e-09 2e-09)
VIN1 na1 0 PULSE(0 1.8 1e-09 20p 20p 2e-09 4e-09)
VIN2 na2 0 PULSE(0 1.8 2e-09 20p 20p 4e-09 8e-09)
VIN3 na3 0 PULSE(0 1.8 4e-09 20p 20p 8e-09 1.6e-08)
VIN4 na4 0 PULSE(0 1.8 8e-09 20p 20p 1.6e-08 3.2e-08)
VIN5 na5 0 PULSE(0 1.8 1.6e-08 20p 20p 3.2e-08 6.4e-08)
VIN6 na6 0 PULSE(0 1.8 3.2e-08 20p 20p 6.4e-08 1.28e-07)
VIN7 na7 0 PULSE(0 1.8 6.4e-08 20p 20p 1.28e-07 2.56e-07)
VIN8 na8 0 PULSE(0 1.8 1.28e-07 20p 20p 2.56e-07 5.12e-07)
VIN9 nb0 0 PULSE(0 1.8 2.56e-07 20p 20p 5.12e-07 1.024e-06)
VIN10 nb1 0 PULSE(0 1.8 5.12e-07 20p 20p 1.024e-06 2.048e-06)
VIN11 nb2 0 PULSE(0 1.8 1.024e-06 20p 20p 2.048e-06 4.096e-06)
VIN12 nb3 0 PULSE(0 1.8 2.048e-06 20p 20p 4.096e-06 8.192e-06)
VIN13 nb4 0 PULSE(0 1.8 4.096e-06 20p 20p 8.192e-06 1.6384e-05)
VIN14 nb5 0 PULSE(0 1.8 8.192e-06 20p 20p 1.6384e-05 3.2768e-05)
VIN15 nb6 0 PULSE(0 1.8 1.6384e-05 20p 20p 3.2768e-05 6.5536e-05)
VIN16 nb7 0 PULSE(0 1.8 3.2768e-05 20p 20p 6.5536e-05 0.000131072)
VIN17 nb8 0 PULSE(0 1.8 6.5536e-05 20p 20p 0.000131072 0.000262144)
VIN18 nop0 0 PULSE(0 1.8 0.000131072 20p 20p 0.000262144 0.000524288)
VIN19 nop1 0 PULSE(0 1.8 0.000262144 20p 20p 0.000524288 0.001048576)
VIN20 ncin 0 PULSE(0 1.8 0.000524288 20p 20p 0.001048576 0.002097152)
M1 nw1 nop0 vdd vdd pch w=2u l=180n
M2 nw1 nop0 0 0 nch w=1u l=180n
Cnw1 nw1 0 2f
M3 nw2 nop1 vdd vdd pch w=2u l=180n
M4 nw2 nop1 0 0 nch w=1u l=180n
Cnw2 nw2 0 2f
CT1 t1 0 0.1f
M5 t1 nw2 vdd vdd pch w=2u l=180n
M6 t1 nw1 vdd vdd pch w=2u l=180n
CT2 t2 0 0.1f
M7 t1 nw2 t2 0 nch w=1u l=180n
M8 t2 nw1 0 0 nch w=1u l=180n
M9 nw3 t1 vdd vdd pch w=2u l=180n
M10 nw3 t1 0 0 nch w=1u l=180n
Cnw3 nw3 0 2f
CT3 t3 0 0.1f
M11 t3 nw2 vdd vdd pch w=2u l=180n
M12 t3 nop0 vdd vdd pch w=2u l=180n
CT4 t4 0 0.1f
M13 t3 nw2 t4 0 nch w=1u l=180n
M14 t4 nop0 0 0 nch w=1u l=180n
M15 nw4 t3 vdd vdd pch w=2u l=180n
M16 nw4 t3 0 0 nch w=1u l=180n
Cnw4 nw4 0 2f
CT5 t5 0 0.1f
M17 t5 nop1 vdd vdd pch w=2u l=180n
M18 t5 nw1 vdd vdd pch w=2u l=180n
CT6 t6 0 0.1f
M19 t5 nop1 t6 0 nch w=1u l=180n
M20 t6 nw1 0 0 nch w=1u l=180n
M21 nw5 t5 vdd vdd pch w=2u l=180n
M22 nw5 t5 0 0 nch w=1u l=180n
Cnw5 nw5 0 2f
CT7 t7 0 0.1f
M23 t7 nop1 vdd vdd pch w=2u l=180n
M24 t7 nop0 vdd vdd pch w=2u l=180n
CT8 t8 0 0.1f
M25 t7 nop1 t8 0 nch w=1u l=180n
M26 t8 nop0 0 0 nch w=1u l=180n
M27 nw6 t7 vdd vdd pch w=2u l=180n
M28 nw6 t7 0 0 nch w=1u l=180n
Cnw6 nw6 0 2f
CT9 t9 0 0.1f
CT10 t10 0 0.1f
CT11 t11 0 0.1f
M29 t9 na0 vdd vdd pch w=2u l=180n
M30 t9 nb0 vdd vdd pch w=2u l=180n
CT12 t12 0 0.1f
M31 t9 na0 t12 0 nch w=1u l=180n
M32 t12 nb0 0 0 nch w=1u l=180n
M33 t10 na0 vdd vdd pch w=2u l=180n
M34 t10 t9 vdd vdd pch w=2u l=180n
CT13 t13 0 0.1f
M35 t10 na0 t13 0 nch w=1u l=180n
M36 t13 t9 0 0 nch w=1u l=180n
M37 t11 nb0 vdd vdd pch w=2u l=180n
M38 t11 t9 vdd vdd pch w=2u l=180n
CT14 t14 0 0.1f
M39 t11 nb0 t14 0 nch w=1u l=180n
M40 t14 t9 0 0 nch w=1u l=180n
M41 nw7 t10 vdd vdd pch w=2u l=180n
M42 nw7 t11 vdd vdd pch w=2u l=180n
CT15 t15 0 0.1f
M43 nw7 t10 t15 0 nch w=1u l=180n
M44 t15 t11 0 0 nch w=1u l=180n
Cnw7 nw7 0 2f
CT16 t16 0 0.1f
CT17 t17 0 0.1f
CT18 t18 0 0.1f
M45 t16 nw7 vdd vdd pch w=2u l=180n
M46 t16 ncin vdd vdd pch w=2u l=180n
CT19 t19 0 0.1f
M47 t16 nw7 t19 0 nch w=1u l=180n
M48 t19 ncin 0 0 nch w=1u l=180n
M49 t17 nw7 vdd vdd pch w=2u l=180n
M50 t17 t16 vdd vdd pch w=2u l=180n
CT20 t20 0 0.1f
M51 t17 nw7 t20 0 nch w=1u l=180n
M52 t20 t16 0 0 nch w=1u l=180n
M53 t18 ncin vdd vdd pch w=2u l=180n
M54 t18 t16 vdd vdd pch w=2u l=180n
CT21 t21 0 0.1f
M55 t18 ncin t21 0 nch w=1u l=180n
M56 t21 t16 0 0 nch w=1u l=180n
M57 nw8 t17 vdd vdd pch w=2u l=180n
M58 nw8 t18 vdd vdd pch w=2u l=180n
CT22 t22 0 0.1f
M59 nw8 t17 t22 0 nch w=1u l=180n
M60 t22 t18 0 0 nch w=1u l=180n
Cnw8 nw8 0 2f
M61 nw9 na0 vdd vdd pch w=2u l=180n
M62 nw9 nb0 vdd vdd pch w=2u l=180n
CT23 t23 0 0.1f
M63 nw9 na0 t23 0 nch w=1u l=180n
M64 t23 nb0 0 0 nch w=1u l=180n
Cnw9 nw9 0 2f
M65 nw10 nw7 vdd vdd pch w=2u l=180n
M66 nw10 ncin vdd vdd pch w=2u l=180n
CT24 t24 0 0.1f
M67 nw10 nw7 t24 0 nch w=1u l=180n
M68 t24 ncin 0 0 nch w=1u l=180n
Cnw10 nw10 0 2f
M69 nw11 nw9 vdd vdd pch w=2u l=180n
M70 nw11 nw10 vdd vdd pch w=2u l=180n
CT25 t25 0 0.1f
M71 nw11 nw9 t25 0 nch w=1u l=180n
M72 t25 nw10 0 0 nch w=1u l=180n
Cnw11 nw11 0 2f
CT26 t26 0 0.1f
M73 t26 na0 vdd vdd pch w=2u l=180n
M74 t26 nb0 vdd vdd pch w=2u l=180n
CT27 t27 0 0.1f
M75 t26 na0 t27 0 nch w=1u l=180n
M76 t27 nb0 0 0 nch w=1u l=180n
M77 nw12 t26 vdd vdd pch w=2u l=180n
M78 nw12 t26 0 0 nch w=1u l=180n
Cnw12 nw12 0 2f
CT28 t28 0 0.1f
M79 t28 na0 0 0 nch w=1u l=180n
M80 t28 nb0 0 0 nch w=1u l=180n
CT29 t29 0 0.1f
M81 t29 na0 vdd vdd pch w=2u l=180n
M82 t28 nb0 t29 vdd pch w=2u l=180n
M83 nw13 t28 vdd vdd pch w=2u l=180n
M84 nw13 t28 0 0 nch w=1u l=180n
Cnw13 nw13 0 2f
CT30 t30 0 0.1f
CT31 t31 0 0.1f
CT32 t32 0 0.1f
M85 t30 na0 vdd vdd pch w=2u l=180n
M86 t30 nb0 vdd vdd pch w=2u l=180n
CT33 t33 0 0.1f
M87 t30 na0 t33 0 nch w=1u l=180n
M88 t33 nb0 0 0 nch w=1u l=180n
M89 t31 na0 vdd vdd pch w=2u l=180n
M90 t31 t30 vdd vdd pch w=2u l=180n
CT34 t34 0 0.1f
M91 t31 na0 t34 0 nch w=1u l=180n
M92 t34 t30 0 0 nch w=1u l=180n
M93 t32 nb0 vdd vdd pch w=2u l=180n
M94 t32 t30 vdd vdd pch w=2u l=180n
CT35 t35 0 0.1f
M95 t32 nb0 t35 0 nch w=1u l=180n
M96 t35 t30 0 0 nch w=1u l=180n
M97 nw14 t31 vdd vdd pch w=2u l=180n
M98 nw14 t32 vdd vdd pch w=2u l=180n
CT36 t36 0 0.1f
M99 nw14 t31 t36 0 nch w=1u l=180n
M100 t36 t32 0 0 nch w=1u l=180n
Cnw14 nw14 0 2f
CT37 t37 0 0.1f
M101 t37 nw12 vdd vdd pch w=2u l=180n
M102 t37 nw3 vdd vdd pch w=2u l=180n
CT38 t38 0 0.1f
M103 t37 nw12 t38 0 nch w=1u l=180n
M104 t38 nw3 0 0 nch w=1u l=180n
M105 nw15 t37 vdd vdd pch w=2u l=180n
M106 nw15 t37 0 0 nch w=1u l=180n
Cnw15 nw15 0 2f
CT39 t39 0 0.1f
M107 t39 nw13 vdd vdd pch w=2u l=180n
M108 t39 nw4 vdd vdd pch w=2u l=180n
CT40 t40 0 0.1f
M109 t39 nw13 t40 0 nch w=1u l=180n
M110 t40 nw4 0 0 nch w=1u l=180n
M111 nw16 t39 vdd vdd pch w=2u l=180n
M112 nw16 t39 0 0 nch w=1u l=180n
Cnw16 nw16 0 2f
CT41 t41 0 0.1f
M113 t41 nw14 vdd vdd pch w=2u l=180n
M114 t41 nw5 vdd vdd pch w=2u l=180n
CT42 t42 0 0.1f
M115 t41 nw14 t42 0 nch w=1u l=180n
M116 t42 nw5 0 0 nch w=1u l=180n
M117 nw17 t41 vdd vdd pch w=2u l=180n
M118 nw17 t41 0 0 nch w=1u l=180n
Cnw17 nw17 0 2f
CT43 t43 0 0.1f
M119 t43 nw8 vdd vdd pch w=2u l=180n
M120 t43 nw6 vdd vdd pch w=2u l=180n
CT44 t44 0 0.1f
M121 t43 nw8 t44 0 nch w=1u l=180n
M122 t44 nw6 0 0 nch w=1u l=180n
M123 nw18 t43 vdd vdd pch w=2u l=180n
M124 nw18 t43 0 0 nch w=1u l=180n
Cnw18 nw18 0 2f
CT45 t45 0 0.1f
M125 t45 nw15 0 0 nch w=1u l=180n
M126 t45 nw16 0 0 nch w=1u l=180n
M127 t45 nw17 0 0 nch w=1u l=180n
M128 t45 nw18 0 0 nch w=1u l=180n
CT46 t46 0 0.1f
M129 t46 nw15 vdd vdd pch w=2u l=180n
CT47 t47 0 0.1f
M130 t47 nw16 t46 vdd pch w=2u l=180n
CT48 t48 0 0.1f
M131 t48 nw17 t47 vdd pch w=2u l=180n
M132 t45 nw18 t48 vdd pch w=2u l=180n
M133 nw19 t45 vdd vdd pch w=2u l=180n
M134 nw19 t45 0 0 nch w=1u l=180n
Cnw19 nw19 0 2f
CT49 t49 0 0.1f
M135 t49 nw19 vdd vdd pch w=2u l=180n
M136 t49 nw19 0 0 nch w=1u l=180n
M137 ny0 t49 vdd vdd pch w=2u l=180n
M138 ny0 t49 0 0 nch w=1u l=180n
Cny0 ny0 0 2f
CT50 t50 0 0.1f
CT51 t51 0 0.1f
CT52 t52 0 0.1f
M139 t50 na1 vdd vdd pch w=2u l=180n
M140 t50 nb1 vdd vdd pch w=2u l=180n
CT53 t53 0 0.1f
M141 t50 na1 t53 0 nch w=1u l=180n
M142 t53 nb1 0 0 nch w=1u l=180n
M143 t51 na1 vdd vdd pch w=2u l=180n
M144 t51 t50 vdd vdd pch w=2u l=180n
CT54 t54 0 0.1f
M145 t51 na1 t54 0 nch w=1u l=180n
M146 t54 t50 0 0 nch w=1u l=180n
M147 t52 nb1 vdd vdd pch w=2u l=180n
M148 t52 t50 vdd vdd pch w=2u l=180n
CT55 t55 0 0.1f
M149 t52 nb1 t55 0 nch w=1u l=180n
M150 t55 t50 0 0 nch w=1u l=180n
M151 nw21 t51 vdd vdd pch w=2u l=180n
M152 nw21 t52 vdd vdd pch w=2u l=180n
CT56 t56 0 0.1f
M153 nw21 t51 t56 0 nch w=1u l=180n
M154 t56 t52 0 0 nch w=1u l=180n
Cnw21 nw21 0 2f
CT57 t57 0 0.1f
CT58 t58 0 0.1f
CT59 t59 0 0.1f
M155 t57 nw21 vdd vdd pch w=2u l=180n
M156 t57 nw11 vdd vdd pch w=2u l=180n
CT60 t60 0 0.1f
M157 t57 nw21 t60 0 nch w=1u l=180n
M158 t60 nw11 0 0 nch w=1u l=180n
M159 t58 nw21 vdd vdd pch w=2u l=180n
M160 t58 t57 vdd vdd pch w=2u l=180n
CT61 t61 0 0.1f
M161 t58 nw21 t61 0 nch w=1u l=180n
M162 t61 t57 0 0 nch w=1u l=180n
M163 t59 nw11 vdd vdd pch w=2u l=180n
M164 t59 t57 vdd vdd pch w=2u l=180n
CT62 t62 0 0.1f
M165 t59 nw11 t62 0 nch w=1u l=180n
M166 t62 t57 0 0 nch w=1u l=180n
M167 nw22 t58 vdd vdd pch w=2u l=180n
M168 nw22 t59 vdd vdd pch w=2u l=180n
CT63 t63 0 0.1f
M169 nw22 t58 t63 0 nch w=1u l=180n
M170 t63 t59 0 0 nch w=1u l=180n
Cnw22 nw22 0 2f
M171 nw23 na1 vdd vdd pch w=2u l=180n
M172 nw23 nb1 vdd vdd pch w=2u l=180n
CT64 t64 0 0.1f
M173 nw23 na1 t64 0 nch w=1u l=180n
M174 t64 nb1 0 0 nch w=1u l=180n
Cnw23 nw23 0 2f
M175 nw24 nw21 vdd vdd pch w=2u l=180n
M176 nw24 nw11 vdd vdd pch w=2u l=180n
CT65 t65 0 0.1f
M177 nw24 nw21 t65 0 nch w=1u l=180n
M178 t65 nw11 0 0 nch w=1u l=180n
Cnw24 nw24 0 2f
M179 nw25 nw23 vdd vdd pch w=2u l=180n
M180 nw25 nw24 vdd vdd pch w=2u l=180n
CT66 t66 0 0.1f
M181 nw25 nw23 t66 0 nch w=1u l=180n
M182 t66 nw24 0 0 nch w=1u l=180n
Cnw25 nw25 0 2f
CT67 t67 0 0.1f
M183 t67 na1 vdd vdd pch w=2u l=180n
M184 t67 nb1 vdd vdd pch w=2u l=180n
CT68 t68 0 0.1f
M185 t67 na1 t68 0 nch w=1u l=180n
M186 t68 nb1 0 0 nch w=1u l=180n
M187 nw26 t67 vdd vdd pch w=2u l=180n
M188 nw26 t67 0 0 nch w=1u l=180n
Cnw26 nw26 0 2f
CT69 t69 0 0.1f
M189 t69 na1 0 0 nch w=1u l=180n
M190 t69 nb1 0 0 nch w=1u l=180n
CT70 t70 0 0.1f
M191 t70 na1 vdd vdd pch w=2u l=180n
M192 t69 nb1 t70 vdd pch w=2u l=180n
M193 nw27 t69 vdd vdd pch w=2u l=180n
M194 nw27 t69 0 0 nch w=1u l=180n
Cnw27 nw27 0 2f
CT71 t71 0 0.1f
CT72 t72 0 0.1f
CT73 t73 0 0.1f
M195 t71 na1 vdd vdd pch w=2u l=180n
M196 t71 nb1 vdd vdd pch w=2u l=180n
CT74 t74 0 0.1f
M197 t71 na1 t74 0 nch w=1u l=180n
M198 t74 nb1 0 0 nch w=1u l=180n
M199 t72 na1 vdd vdd pch w=2u l=180n
M200 t72 t71 vdd vdd pch w=2u l=180n
CT75 t75 0 0.1f
M201 t72 na1 t75 0 nch w=1u l=180n
M202 t75 t71 0 0 nch w=1u l=180n
M203 t73 nb1 vdd vdd pch w=2u l=180n
M204 t73 t71 vdd vdd pch w=2u l=180n
CT76 t76 0 0.1f
M205 t73 nb1 t76 0 nch w=1u l=180n
M206 t76 t71 0 0 nch w=1u l=180n
M207 nw28 t72 vdd vdd pch w=2u l=180n
M208 nw28 t73 vdd vdd pch w=2u l=180n
CT77 t77 0 0.1f
M209 nw28 t72 t77 0 nch w=1u l=180n
M210 t77 t73 0 0 nch w=1u l=180n
Cnw28 nw28 0 2f
CT78 t78 0 0.1f
M211 t78 nw26 vdd vdd pch w=2u l=180n
M212 t78 nw3 vdd vdd pch w=2u l=180n
CT79 t79 0 0.1f
M213 t78 nw26 t79 0 nch w=1u l=180n
M214 t79 nw3 0 0 nch w=1u l=180n
M215 nw29 t78 vdd vdd pch w=2u l=180n
M216 nw29 t78 0 0 nch w=1u l=180n
Cnw29 nw29 0 2f
CT80 t80 0 0.1f
M217 t80 nw27 vdd vdd pch w=2u l=180n
M218 t80 nw4 vdd vdd pch w=2u l=180n
CT81 t81 0 0.1f
M219 t80 nw27 t81 0 nch w=1u l=180n
M220 t81 nw4 0 0 nch w=1u l=180n
M221 nw30 t80 vdd vdd pch w=2u l=180n
M222 nw30 t80 0 0 nch w=1u l=180n
Cnw30 nw30 0 2f
CT82 t82 0 0.1f
M223 t82 nw28 vdd vdd pch w=2u l=180n
M224 t82 nw5 vdd vdd pch w=2u l=180n
CT83 t83 0 0.1f
M225 t82 nw28 t83 0 nch w=1u l=180n
M226 t83 nw5 0 0 nch w=1u l=180n
M227 nw31 t82 vdd vdd pch w=2u l=180n
M228 nw31 t82 0 0 nch w=1u l=180n
Cnw31 nw31 0 2f
CT84 t84 0 0.1f
M229 t84 nw22 vdd vdd pch w=2u l=180n
M230 t84 nw6 vdd vdd pch w=2u l=180n
CT85 t85 0 0.1f
M231 t84 nw22 t85 0 nch w=1u l=180n
M232 t85 nw6 0 0 nch w=1u l=180n
M233 nw32 t84 vdd vdd pch w=2u l=180n
M234 nw32 t84 0 0 nch w=1u l=180n
Cnw32 nw32 0 2f
CT86 t86 0 0.1f
M235 t86 nw29 0 0 nch w=1u l=180n
M236 t86 nw30 0 0 nch w=1u l=180n
M237 t86 nw31 0 0 nch w=1u l=180n
M238 t86 nw32 0 0 nch w=1u l=180n
CT87 t87 0 0.1f
M239 t87 nw29 vdd vdd pch w=2u l=180n
CT88 t88 0 0.1f
M240 t88 nw30 t87 vdd pch w=2u l=180n
CT89 t89 0 0.1f
M241 t89 nw31 t88 vdd pch w=2u l=180n
M242 t86 nw32 t89 vdd pch w=2u l=180n
M243 nw33 t86 vdd vdd pch w=2u l=180n
M244 nw33 t86 0 0 nch w=1u l=180n
Cnw33 nw33 0 2f
CT90 t90 0 0.1f
M245 t90 nw33 vdd vdd pch w=2u l=180n
M246 t90 nw33 0 0 nch w=1u l=180n
M247 ny1 t90 vdd vdd pch w=2u l=180n
M248 ny1 t90 0 0 nch w=1u l=180n
Cny1 ny1 0 2f
CT91 t91 0 0.1f
CT92 t92 0 0.1f
CT93 t93 0 0.1f
M249 t91 na2 vdd vdd pch w=2u l=180n
M250 t91 nb2 vdd vdd pch w=2u l=180n
CT94 t94 0 0.1f
M251 t91 na2 t94 0 nch w=1u l=180n
M252 t94 nb2 0 0 nch w=1u l=180n
M253 t92 na2 vdd vdd pch w=2u l=180n
M254 t92 t91 vdd vdd pch w=2u l=180n
CT95 t95 0 0.1f
M255 t92 na2 t95 0 nch w=1u l=180n
M256 t95 t91 0 0 nch w=1u l=180n
M257 t93 nb2 vdd vdd pch w=2u l=180n
M258 t93 t91 vdd vdd pch w=2u l=180n
CT96 t96 0 0.1f
M259 t93 nb2 t96 0 nch w=1u l=180n
M260 t96 t91 0 0 nch w=1u l=180n
M261 nw35 t92 vdd vdd pch w=2u l=180n
M262 nw35 t93 vdd vdd pch w=2u l=180n
CT97 t97 0 0.1f
M263 nw35 t92 t97 0 nch w=1u l=180n
M264 t97 t93 0 0 nch w=1u l=180n
Cnw35 nw35 0 2f
CT98 t98 0 0.1f
CT99 t99 0 0.1f
CT100 t100 0 0.1f
M265 t98 nw35 vdd vdd pch w=2u l=180n
M266 t98 nw25 vdd vdd pch w=2u l=180n
CT101 t101 0 0.1f
M267 t98 nw35 t101 0 nch w=1u l=180n
M268 t101 nw25 0 0 nch w=1u l=180n
M269 t99 nw35 vdd vdd pch w=2u l=180n
M270 t99 t98 vdd vdd pch w=2u l=180n
CT102 t102 0 0.1f
M271 t99 nw35 t102 0 nch w=1u l=180n
M272 t102 t98 0 0 nch w=1u l=180n
M273 t100 nw25 vdd vdd pch w=2u l=180n
M274 t100 t98 vdd vdd pch w=2u l=180n
CT103 t103 0 0.1f
M275 t100 nw25 t103 0 nch w=1u l=180n
M276 t103 t98 0 0 nch w=1u l=180n
M277 nw36 t99 vdd vdd pch w=2u l=180n
M278 nw36 t100 vdd vdd pch w=2u l=180n
CT104 t104 0 0.1f
M279 nw36 t99 t104 0 nch w=1u l=180n
M280 t104 t100 0 0 nch w=1u l=180n
Cnw36 nw36 0 2f
M281 nw37 na2 vdd vdd pch w=2u l=180n
M282 nw37 nb2 vdd vdd pch w=2u l=180n
CT105 t105 0 0.1f
M283 nw37 na2 t105 0 nch w=1u l=180n
M284 t105 nb2 0 0 nch w=1u l=180n
Cnw37 nw37 0 2f
M285 nw38 nw35 vdd vdd pch w=2u l=180n
M286 nw38 nw25 vdd vdd pch w=2u l=180n
CT106 t106 0 0.1f
M287 nw38 nw35 t106 0 nch w=1u l=180n
M288 t106 nw25 0 0 nch w=1u l=180n
Cnw38 nw38 0 2f
M289 nw39 nw37 vdd vdd pch w=2u l=180n
M290 nw39 nw38 vdd vdd pch w=2u l=180n
CT107 t107 0 0.1f
M291 nw39 nw37 t107 0 nch w=1u l=180n
M292 t107 nw38 0 0 nch w=1u l=180n
Cnw39 nw39 0 2f
CT108 t108 0 0.1f
M293 t108 na2 vdd vdd pch w=2u l=180n
M294 t108 nb2 vdd vdd pch w=2u l=180n
CT109 t109 0 0.1f
M295 t108 na2 t109 0 nch w=1u l=180n
M296 t109 nb2 0 0 nch w=1u l=180n
M297 nw40 t108 vdd vdd pch w=2u l=180n
M298 nw40 t108 0 0 nch w=1u l=180n
Cnw40 nw40 0 2f
CT110 t110 0 0.1f
M299 t110 na2 0 0 nch w=1u l=180n
M300 t110 nb2 0 0 nch w=1u l=180n
CT111 t111 0 0.1f
M301 t111 na2 vdd vdd pch w=2u l=180n
M302 t110 nb2 t111 vdd pch w=2u l=180n
M303 nw41 t110 vdd vdd pch w=2u l=180n
M304 nw41 t110 0 0 nch w=1u l=180n
Cnw41 nw41 0 2f
CT112 t112 0 0.1f
CT113 t113 0 0.1f
CT114 t114 0 0.1f
M305 t112 na2 vdd vdd pch w=2u l=180n
M306 t112 nb2 vdd vdd pch w=2u l=180n
CT115 t115 0 0.1f
M307 t112 na2 t115 0 nch w=1u l=180n
M308 t115 nb2 0 0 nch w=1u l=180n
M309 t113 na2 vdd vdd pch w=2u l=180n
M310 t113 t112 vdd vdd pch w=2u l=180n
CT116 t116 0 0.1f
M311 t113 na2 t116 0 nch w=1u l=180n
M312 t116 t112 0 0 nch w=1u l=180n
M313 t114 nb2 vdd vdd pch w=2u l=180n
M314 t114 t112 vdd vdd pch w=2u l=180n
CT117 t117 0 0.1f
M315 t114 nb2 t117 0 nch w=1u l=180n
M316 t117 t112 0 0 nch w=1u l=180n
M317 nw42 t113 vdd vdd pch w=2u l=180n
M318 nw42 t114 vdd vdd pch w=2u l=180n
CT118 t118 0 0.1f
M319 nw42 t113 t118 0 nch w=1u l=180n
M320 t118 t114 0 0 nch w=1u l=180n
Cnw42 nw42 0 2f
CT119 t119 0 0.1f
M321 t119 nw40 vdd vdd pch w=2u l=180n
M322 t119 nw3 vdd vdd pch w=2u l=180n
CT120 t120 0 0.1f
M323 t119 nw40 t120 0 nch w=1u l=180n
M324 t120 nw3 0 0 nch w=1u l=180n
M325 nw43 t119 vdd vdd pch w=2u l=180n
M326 nw43 t119 0 0 nch w=1u l=180n
Cnw43 nw43 0 2f
CT121 t121 0 0.1f
M327 t121 nw41 vdd vdd pch w=2u l=180n
M328 t121 nw4 vdd vdd pch w=2u l=180n
CT122 t122 0 0.1f
M329 t121 nw41 t122 0 nch w=1u l=180n
M330 t122 nw4 0 0 nch w=1u l=180n
M331 nw44 t121 vdd vdd pch w=2u l=180n
M332 nw44 t121 0 0 nch w=1u l=180n
Cnw44 nw44 0 2f
CT123 t123 0 0.1f
M333 t123 nw42 vdd vdd pch w=2u l=180n
M334 t123 nw5 vdd vdd pch w=2u l=180n
CT124 t124 0 0.1f
M335 t123 nw42 t124 0 nch w=1u l=180n
M336 t124 nw5 0 0 nch w=1u l=180n
M337 nw45 t123 vdd vdd pch w=2u l=180n
M338 nw45 t123 0 0 nch w=1u l=180n
Cnw45 nw45 0 2f
CT125 t125 0 0.1f
M339 t125 nw36 vdd vdd pch w=2u l=180n
M340 t125 nw6 vdd vdd pch w=2u l=180n
CT126 t126 0 0.1f
M341 t125 nw36 t126 0 nch w=1u l=180n
M342 t126 nw6 0 0 nch w=1u l=180n
M343 nw46 t125 vdd vdd pch w=2u l=180n
M344 nw46 t125 0 0 nch w=1u l=180n
Cnw46 nw46 0 2f
CT127 t127 0 0.1f
M345 t127 nw43 0 0 nch w=1u l=180n
M346 t127 nw44 0 0 nch w=1u l=180n
M347 t127 nw45 0 0 nch w=1u l=180n
M348 t127 nw46 0 0 nch w=1u l=180n
CT128 t128 0 0.1f
M349 t128 nw43 vdd vdd pch w=2u l=180n
CT129 t129 0 0.1f
M350 t129 nw44 t128 vdd pch w=2u l=180n
CT130 t130 0 0.1f
M351 t130 nw45 t129 vdd pch w=2u l=180n
M352 t127 nw46 t130 vdd pch w=2u l=180n
M353 nw47 t127 vdd vdd pch w=2u l=180n
M354 nw47 t127 0 0 nch w=1u l=180n
Cnw47 nw47 0 2f
CT131 t131 0 0.1f
M355 t131 nw47 vdd vdd pch w=2u l=180n
M356 t131 nw47 0 0 nch w=1u l=180n
M357 ny2 t131 vdd vdd pch w=2u l=180n
M358 ny2 t131 0 0 nch w=1u l=180n
Cny2 ny2 0 2f
CT132 t132 0 0.1f
CT133 t133 0 0.1f
CT134 t134 0 0.1f
M359 t132 na3 vdd vdd pch w=2u l=180n
M360 t132 nb3 vdd vdd pch w=2u l=180n
CT135 t135 0 0.1f
M361 t132 na3 t135 0 nch w=1u l=180n
M362 t135 nb3 0 0 nch w=1u l=180n
M363 t133 na3 vdd vdd pch w=2u l=180n
M364 t133 t132 vdd vdd pch w=2u l=180n
CT136 t136 0 0.1f
M365 t133 na3 t136 0 nch w=1u l=180n
M366 t136 t132 0 0 nch w=1u l=180n
M367 t134 nb3 vdd vdd pch w=2u l=180n
M368 t134 t132 vdd vdd pch w=2u l=180n
CT137 t137 0 0.1f
M369 t134 nb3 t137 0 nch w=1u l=180n
M370 t137 t132 0 0 nch w=1u l=180n
M371 nw49 t133 vdd vdd pch w=2u l=180n
M372 nw49 t134 vdd vdd pch w=2u l=180n
CT138 t138 0 0.1f
M373 nw49 t133 t138 0 nch w=1u l=180n
M374 t138 t134 0 0 nch w=1u l=180n
Cnw49 nw49 0 2f
CT139 t139 0 0.1f
CT140 t140 0 0.1f
CT141 t141 0 0.1f
M375 t139 nw49 vdd vdd pch w=2u l=180n
M376 t139 nw39 vdd vdd pch w=2u l=180n
CT142 t142 0 0.1f
M377 t139 nw49 t142 0 nch w=1u l=180n
M378 t142 nw39 0 0 nch w=1u l=180n
M379 t140 nw49 vdd vdd pch w=2u l=180n
M380 t140 t139 vdd vdd pch w=2u l=180n
CT143 t143 0 0.1f
M381 t140 nw49 t143 0 nch w=1u l=180n
M382 t143 t139 0 0 nch w=1u l=180n
M383 t141 nw39 vdd vdd pch w=2u l=180n
M384 t141 t139 vdd vdd pch w=2u l=180n
CT144 t144 0 0.1f
M385 t141 nw39 t144 0 nch w=1u l=180n
M386 t144 t139 0 0 nch w=1u l=180n
M387 nw50 t140 vdd vdd pch w=2u l=180n
M388 nw50 t141 vdd vdd pch w=2u l=180n
CT145 t145 0 0.1f
M389 nw50 t140 t145 0 nch w=1u l=180n
M390 t145 t141 0 0 nch w=1u l=180n
Cnw50 nw50 0 2f
M391 nw51 na3 vdd vdd pch w=2u l=180n
M392 nw51 nb3 vdd vdd pch w=2u l=180n
CT146 t146 0 0.1f
M393 nw51 na3 t146 0 nch w=1u l=180n
M394 t146 nb3 0 0 nch w=1u l=180n
Cnw51 nw51 0 2f
M395 nw52 nw49 vdd vdd pch w=2u l=180n
M396 nw52 nw39 vdd vdd pch w=2u l=180n
CT147 t147 0 0.1f
M397 nw52 nw49 t147 0 nch w=1u l=180n
M398 t147 nw39 0 0 nch w=1u l=180n
Cnw52 nw52 0 2f
M399 nw53 nw51 vdd vdd pch w=2u l=180n
M400 nw53 nw52 vdd vdd pch w=2u l=180n
CT148 t148 0 0.1f
M401 nw53 nw51 t148 0 nch w=1u l=180n
M402 t148 nw52 0 0 nch w=1u l=180n
Cnw53 nw53 0 2f
CT149 t149 0 0.1f
M403 t149 na3 vdd vdd pch w=2u l=180n
M404 t149 nb3 vdd vdd pch w=2u l=180n
CT150 t150 0 0.1f
M405 t149 na3 t150 0 nch w=1u l=180n
M406 t150 nb3 0 0 nch w=1u l=180n
M407 nw54 t149 vdd vdd pch w=2u l=180n
M408 nw54 t149 0 0 nch w=1u l=180n
Cnw54 nw54 0 2f
CT151 t151 0 0.1f
M409 t151 na3 0 0 nch w=1u l=180n
M410 t151 nb3 0 0 nch w=1u l=180n
CT152 t152 0 0.1f
M411 t152 na3 vdd vdd pch w=2u l=180n
M412 t151 nb3 t152 vdd pch w=2u l=180n
M413 nw55 t151 vdd vdd pch w=2u l=180n
M414 nw55 t151 0 0 nch w=1u l=180n
Cnw55 nw55 0 2f
CT153 t153 0 0.1f
CT154 t154 0 0.1f
CT155 t155 0 0.1f
M415 t153 na3 vdd vdd pch w=2u l=180n
M416 t153 nb3 vdd vdd pch w=2u l=180n
CT156 t156 0 0.1f
M417 t153 na3 t156 0 nch w=1u l=180n
M418 t156 nb3 0 0 nch w=1u l=180n
M419 t154 na3 vdd vdd pch w=2u l=180n
M420 t154 t153 vdd vdd pch w=2u l=180n
CT157 t157 0 0.1f
M421 t154 na3 t157 0 nch w=1u l=180n
M422 t157 t153 0 0 nch w=1u l=180n
M423 t155 nb3 vdd vdd pch w=2u l=180n
M424 t155 t153 vdd vdd pch w=2u l=180n
CT158 t158 0 0.1f
M425 t155 nb3 t158 0 nch w=1u l=180n
M426 t158 t153 0 0 nch w=1u l=180n
M427 nw56 t154 vdd vdd pch w=2u l=180n
M428 nw56 t155 vdd vdd pch w=2u l=180n
CT159 t159 0 0.1f
M429 nw56 t154 t159 0 nch w=1u l=180n
M430 t159 t155 0 0 nch w=1u l=180n
Cnw56 nw56 0 2f
CT160 t160 0 0.1f
M431 t160 nw54 vdd vdd pch w=2u l=180n
M432 t160 nw3 vdd vdd pch w=2u l=180n
CT161 t161 0 0.1f
M433 t160 nw54 t161 0 nch w=1u l=180n
M434 t161 nw3 0 0 nch w=1u l=180n
M435 nw57 t160 vdd vdd pch w=2u l=180n
M436 nw57 t160 0 0 nch w=1u l=180n
Cnw57 nw57 0 2f
CT162 t162 0 0.1f
M437 t162 nw55 vdd vdd pch w=2u l=180n
M438 t162 nw4 vdd vdd pch w=2u l=180n
CT163 t163 0 0.1f
M439 t162 nw55 t163 0 nch w=1u l=180n
M440 t163 nw4 0 0 nch w=1u l=180n
M441 nw58 t162 vdd vdd pch w=2u l=180n
M442 nw58 t162 0 0 nch w=1u l=180n
Cnw58 nw58 0 2f
CT164 t164 0 0.1f
M443 t164 nw56 vdd vdd pch w=2u l=180n
M444 t164 nw5 vdd vdd pch w=2u l=180n
CT165 t165 0 0.1f
M445 t164 nw56 t165 0 nch w=1u l=180n
M446 t165 nw5 0 0 nch w=1u l=180n
M447 nw59 t164 vdd vdd pch w=2u l=180n
M448 nw59 t164 0 0 nch w=1u l=180n
Cnw59 nw59 0 2f
CT166 t166 0 0.1f
M449 t166 nw50 vdd vdd pch w=2u l=180n
M450 t166 nw6 vdd vdd pch w=2u l=180n
CT167 t167 0 0.1f
M451 t166 nw50 t167 0 nch w=1u l=180n
M452 t167 nw6 0 0 nch w=1u l=180n
M453 nw60 t166 vdd vdd pch w=2u l=180n
M454 nw60 t166 0 0 nch w=1u l=180n
Cnw60 nw60 0 2f
CT168 t168 0 0.1f
M455 t168 nw57 0 0 nch w=1u l=180n
M456 t168 nw58 0 0 nch w=1u l=180n
M457 t168 nw59 0 0 nch w=1u l=180n
M458 t168 nw60 0 0 nch w=1u l=180n
CT169 t169 0 0.1f
M459 t169 nw57 vdd vdd pch w=2u l=180n
CT170 t170 0 0.1f
M460 t170 nw58 t169 vdd pch w=2u l=180n
CT171 t171 0 0.1f
M461 t171 nw59 t170 vdd pch w=2u l=180n
M462 t168 nw60 t171 vdd pch w=2u l=180n
M463 nw61 t168 vdd vdd pch w=2u l=180n
M464 nw61 t168 0 0 nch w=1u l=180n
Cnw61 nw61 0 2f
CT172 t172 0 0.1f
M465 t172 nw61 vdd vdd pch w=2u l=180n
M466 t172 nw61 0 0 nch w=1u l=180n
M467 ny3 t172 vdd vdd pch w=2u l=180n
M468 ny3 t172 0 0 nch w=1u l=180n
Cny3 ny3 0 2f
CT173 t173 0 0.1f
CT174 t174 0 0.1f
CT175 t175 0 0.1f
M469 t173 na4 vdd vdd pch w=2u l=180n
M470 t173 nb4 vdd vdd pch w=2u l=180n
CT176 t176 0 0.1f
M471 t173 na4 t176 0 nch w=1u l=180n
M472 t176 nb4 0 0 nch w=1u l=180n
M473 t174 na4 vdd vdd pch w=2u l=180n
M474 t174 t173 vdd vdd pch w=2u l=180n
CT177 t177 0 0.1f
M475 t174 na4 t177 0 nch w=1u l=180n
M476 t177 t173 0 0 nch w=1u l=180n
M477 t175 nb4 vdd vdd pch w=2u l=180n
M478 t175 t173 vdd vdd pch w=2u l=180n
CT178 t178 0 0.1f
M479 t175 nb4 t178 0 nch w=1u l=180n
M480 t178 t173 0 0 nch w=1u l=180n
M481 nw63 t174 vdd vdd pch w=2u l=180n
M482 nw63 t175 vdd vdd pch w=2u l=180n
CT179 t179 0 0.1f
M483 nw63 t174 t179 0 nch w=1u l=180n
M484 t179 t175 0 0 nch w=1u l=180n
Cnw63 nw63 0 2f
CT180 t180 0 0.1f
CT181 t181 0 0.1f
CT182 t182 0 0.1f
M485 t180 nw63 vdd vdd pch w=2u l=180n
M486 t180 nw53 vdd vdd pch w=2u l=180n
CT183 t183 0 0.1f
M487 t180 nw63 t183 0 nch w=1u l=180n
M488 t183 nw53 0 0 nch w=1u l=180n
M489 t181 nw63 vdd vdd pch w=2u l=180n
M490 t181 t180 vdd vdd pch w=2u l=180n
CT184 t184 0 0.1f
M491 t181 nw63 t184 0 nch w=1u l=180n
M492 t184 t180 0 0 nch w=1u l=180n
M493 t182 nw53 vdd vdd pch w=2u l=180n
M494 t182 t180 vdd vdd pch w=2u l=180n
CT185 t185 0 0.1f
M495 t182 nw53 t185 0 nch w=1u l=180n
M496 t185 t180 0 0 nch w=1u l=180n
M497 nw64 t181 vdd vdd pch w=2u l=180n
M498 nw64 t182 vdd vdd pch w=2u l=180n
CT186 t186 0 0.1f
M499 nw64 t181 t186 0 nch w=1u l=180n
M500 t186 t182 0 0 nch w=1u l=180n
Cnw64 nw64 0 2f
M501 nw65 na4 vdd vdd pch w=2u l=180n
M502 nw65 nb4 vdd vdd pch w=2u l=180n
CT187 t187 0 0.1f
M503 nw65 na4 t187 0 nch w=1u l=180n
M504 t187 nb4 0 0 nch w=1u l=180n
Cnw65 nw65 0 2f
M505 nw66 nw63 vdd vdd pch w=2u l=180n
M506 nw66 nw53 vdd vdd pch w=2u l=180n
CT188 t188 0 0.1f
M507 nw66 nw63 t188 0 nch w=1u l=180n
M508 t188 nw53 0 0 nch w=1u l=180n
Cnw66 nw66 0 2f
M509 nw67 nw65 vdd vdd pch w=2u l=180n
M510 nw67 nw66 vdd vdd pch w=2u l=180n
CT189 t189 0 0.1f
M511 nw67 nw65 t189 0 nch w=1u l=180n
M512 t189 nw66 0 0 nch w=1u l=180n
Cnw67 nw67 0 2f
CT190 t190 0 0.1f
M513 t190 na4 vdd vdd pch w=2u l=180n
M514 t190 nb4 vdd vdd pch w=2u l=180n
CT191 t191 0 0.1f
M515 t190 na4 t191 0 nch w=1u l=180n
M516 t191 nb4 0 0 nch w=1u l=180n
M517 nw68 t190 vdd vdd pch w=2u l=180n
M518 nw68 t190 0 0 nch w=1u l=180n
Cnw68 nw68 0 2f
CT192 t192 0 0.1f
M519 t192 na4 0 0 nch w=1u l=180n
M520 t192 nb4 0 0 nch w=1u l=180n
CT193 t193 0 0.1f
M521 t193 na4 vdd vdd pch w=2u l=180n
M522 t192 nb4 t193 vdd pch w=2u l=180n
M523 nw69 t192 vdd vdd pch w=2u l=180n
M524 nw69 t192 0 0 nch w=1u l=180n
Cnw69 nw69 0 2f
CT194 t194 0 0.1f
CT195 t195 0 0.1f
CT196 t196 0 0.1f
M525 t194 na4 vdd vdd pch w=2u l=180n
M526 t194 nb4 vdd vdd pch w=2u l=180n
CT197 t197 0 0.1f
M527 t194 na4 t197 0 nch w=1u l=180n
M528 t197 nb4 0 0 nch w=1u l=180n
M529 t195 na4 vdd vdd pch w=2u l=180n
M530 t195 t194 vdd vdd pch w=2u l=180n
CT198 t198 0 0.1f
M531 t195 na4 t198 0 nch w=1u l=180n
M532 t198 t194 0 0 nch w=1u l=180n
M533 t196 nb4 vdd vdd pch w=2u l=180n
M534 t196 t194 vdd vdd pch w=2u l=180n
CT199 t199 0 0.1f
M535 t196 nb4 t199 0 nch w=1u l=180n
M536 t199 t194 0 0 nch w=1u l=180n
M537 nw70 t195 vdd vdd pch w=2u l=180n
M538 nw70 t196 vdd vdd pch w=2u l=180n
CT200 t200 0 0.1f
M539 nw70 t195 t200 0 nch w=1u l=180n
M540 t200 t196 0 0 nch w=1u l=180n
Cnw70 nw70 0 2f
CT201 t201 0 0.1f
M541 t201 nw68 vdd vdd pch w=2u l=180n
M542 t201 nw3 vdd vdd pch w=2u l=180n
CT202 t202 0 0.1f
M543 t201 nw68 t202 0 nch w=1u l=180n
M544 t202 nw3 0 0 nch w=1u l=180n
M545 nw71 t201 vdd vdd pch w=2u l=180n
M546 nw71 t201 0 0 nch w=1u l=180n
Cnw71 nw71 0 2f
CT203 t203 0 0.1f
M547 t203 nw69 vdd vdd pch w=2u l=180n
M548 t203 nw4 vdd vdd pch w=2u l=180n
CT204 t204 0 0.1f
M549 t203 nw69 t204 0 nch w=1u l=180n
M550 t204 nw4 0 0 nch w=1u l=180n
M551 nw72 t203 vdd vdd pch w=2u l=180n
M552 nw72 t203 0 0 nch w=1u l=180n
Cnw72 nw72 0 2f
CT205 t205 0 0.1f
M553 t205 nw70 vdd vdd pch w=2u l=180n
M554 t205 nw5 vdd vdd pch w=2u l=180n
CT206 t206 0 0.1f
M555 t205 nw70 t206 0 nch w=1u l=180n
M556 t206 nw5 0 0 nch w=1u l=180n
M557 nw73 t205 vdd vdd pch w=2u l=180n
M558 nw73 t205 0 0 nch w=1u l=180n
Cnw73 nw73 0 2f
CT207 t207 0 0.1f
M559 t207 nw64 vdd vdd pch w=2u l=180n
M560 t207 nw6 vdd vdd pch w=2u l=180n
CT208 t208 0 0.1f
M561 t207 nw64 t208 0 nch w=1u l=180n
M562 t208 nw6 0 0 nch w=1u l=180n
M563 nw74 t207 vdd vdd pch w=2u l=180n
M564 nw74 t207 0 0 nch w=1u l=180n
Cnw74 nw74 0 2f
CT209 t209 0 0.1f
M565 t209 nw71 0 0 nch w=1u l=180n
M566 t209 nw72 0 0 nch w=1u l=180n
M567 t209 nw73 0 0 nch w=1u l=180n
M568 t209 nw74 0 0 nch w=1u l=180n
CT210 t210 0 0.1f
M569 t210 nw71 vdd vdd pch w=2u l=180n
CT211 t211 0 0.1f
M570 t211 nw72 t210 vdd pch w=2u l=180n
CT212 t212 0 0.1f
M571 t212 nw73 t211 vdd pch w=2u l=180n
M572 t209 nw74 t212 vdd pch w=2u l=180n
M573 nw75 t209 vdd vdd pch w=2u l=180n
M574 nw75 t209 0 0 nch w=1u l=180n
Cnw75 nw75 0 2f
CT213 t213 0 0.1f
M575 t213 nw75 vdd vdd pch w=2u l=180n
M576 t213 nw75 0 0 nch w=1u l=180n
M577 ny4 t213 vdd vdd pch w=2u l=180n
M578 ny4 t213 0 0 nch w=1u l=180n
Cny4 ny4 0 2f
CT214 t214 0 0.1f
CT215 t215 0 0.1f
CT216 t216 0 0.1f
M579 t214 na5 vdd vdd pch w=2u l=180n
M580 t214 nb5 vdd vdd pch w=2u l=180n
CT217 t217 0 0.1f
M581 t214 na5 t217 0 nch w=1u l=180n
M582 t217 nb5 0 0 nch w=1u l=180n
M583 t215 na5 vdd vdd pch w=2u l=180n
M584 t215 t214 vdd vdd pch w=2u l=180n
CT218 t218 0 0.1f
M585 t215 na5 t218 0 nch w=1u l=180n
M586 t218 t214 0 0 nch w=1u l=180n
M587 t216 nb5 vdd vdd pch w=2u l=180n
M588 t216 t214 vdd vdd pch w=2u l=180n
CT219 t219 0 0.1f
M589 t216 nb5 t219 0 nch w=1u l=180n
M590 t219 t214 0 0 nch w=1u l=180n
M591 nw77 t215 vdd vdd pch w=2u l=180n
M592 nw77 t216 vdd vdd pch w=2u l=180n
CT220 t220 0 0.1f
M593 nw77 t215 t220 0 nch w=1u l=180n
M594 t220 t216 0 0 nch w=1u l=180n
Cnw77 nw77 0 2f
CT221 t221 0 0.1f
CT222 t222 0 0.1f
CT223 t223 0 0.1f
M595 t221 nw77 vdd vdd pch w=2u l=180n
M596 t221 nw67 vdd vdd pch w=2u l=180n
CT224 t224 0 0.1f
M597 t221 nw77 t224 0 nch w=1u l=180n
M598 t224 nw67 0 0 nch w=1u l=180n
M599 t222 nw77 vdd vdd pch w=2u l=180n
M600 t222 t221 vdd vdd pch w=2u l=180n
CT225 t225 0 0.1f
M601 t222 nw77 t225 0 nch w=1u l=180n
M602 t225 t221 0 0 nch w=1u l=180n
M603 t223 nw67 vdd vdd pch w=2u l=180n
M604 t223 t221 vdd vdd pch w=2u l=180n
CT226 t226 0 0.1f
M605 t223 nw67 t226 0 nch w=1u l=180n
M606 t226 t221 0 0 nch w=1u l=180n
M607 nw78 t222 vdd vdd pch w=2u l=180n
M608 nw78 t223 vdd vdd pch w=2u l=180n
CT227 t227 0 0.1f
M609 nw78 t222 t227 0 nch w=1u l=180n
M610 t227 t223 0 0 nch w=1u l=180n
Cnw78 nw78 0 2f
M611 nw79 na5 vdd vdd pch w=2u l=180n
M612 nw79 nb5 vdd vdd pch w=2u l=180n
CT228 t228 0 0.1f
M613 nw79 na5 t228 0 nch w=1u l=180n
M614 t228 nb5 0 0 nch w=1u l=180n
Cnw79 nw79 0 2f
M615 nw80 nw77 vdd vdd pch w=2u l=180n
M616 nw80 nw67 vdd vdd pch w=2u l=180n
CT229 t229 0 0.1f
M617 nw80 nw77 t229 0 nch w=1u l=180n
M618 t229 nw67 0 0 nch w=1u l=180n
Cnw80 nw80 0 2f
M619 nw81 nw79 vdd vdd pch w=2u l=180n
M620 nw81 nw80 vdd vdd pch w=2u l=180n
CT230 t230 0 0.1f
M621 nw81 nw79 t230 0 nch w=1u l=180n
M622 t230 nw80 0 0 nch w=1u l=180n
Cnw81 nw81 0 2f
CT231 t231 0 0.1f
M623 t231 na5 vdd vdd pch w=2u l=180n
M624 t231 nb5 vdd vdd pch w=2u l=180n
CT232 t232 0 0.1f
M625 t231 na5 t232 0 nch w=1u l=180n
M626 t232 nb5 0 0 nch w=1u l=180n
M627 nw82 t231 vdd vdd pch w=2u l=180n
M628 nw82 t231 0 0 nch w=1u l=180n
Cnw82 nw82 0 2f
CT233 t233 0 0.1f
M629 t233 na5 0 0 nch w=1u l=180n
M630 t233 nb5 0 0 nch w=1u l=180n
CT234 t234 0 0.1f
M631 t234 na5 vdd vdd pch w=2u l=180n
M632 t233 nb5 t234 vdd pch w=2u l=180n
M633 nw83 t233 vdd vdd pch w=2u l=180n
M634 nw83 t233 0 0 nch w=1u l=180n
Cnw83 nw83 0 2f
CT235 t235 0 0.1f
CT236 t236 0 0.1f
CT237 t237 0 0.1f
M635 t235 na5 vdd vdd pch w=2u l=180n
M636 t235 nb5 vdd vdd pch w=2u l=180n
CT238 t238 0 0.1f
M637 t235 na5 t238 0 nch w=1u l=180n
M638 t238 nb5 0 0 nch w=1u l=180n
M639 t236 na5 vdd vdd pch w=2u l=180n
M640 t236 t235 vdd vdd pch w=2u l=180n
CT239 t239 0 0.1f
M641 t236 na5 t239 0 nch w=1u l=180n
M642 t239 t235 0 0 nch w=1u l=180n
M643 t237 nb5 vdd vdd pch w=2u l=180n
M644 t237 t235 vdd vdd pch w=2u l=180n
CT240 t240 0 0.1f
M645 t237 nb5 t240 0 nch w=1u l=180n
M646 t240 t235 0 0 nch w=1u l=180n
M647 nw84 t236 vdd vdd pch w=2u l=180n
M648 nw84 t237 vdd vdd pch w=2u l=180n
CT241 t241 0 0.1f
M649 nw84 t236 t241 0 nch w=1u l=180n
M650 t241 t237 0 0 nch w=1u l=180n
Cnw84 nw84 0 2f
CT242 t242 0 0.1f
M651 t242 nw82 vdd vdd pch w=2u l=180n
M652 t242 nw3 vdd vdd pch w=2u l=180n
CT243 t243 0 0.1f
M653 t242 nw82 t243 0 nch w=1u l=180n
M654 t243 nw3 0 0 nch w=1u l=180n
M655 nw85 t242 vdd vdd pch w=2u l=180n
M656 nw85 t242 0 0 nch w=1u l=180n
Cnw85 nw85 0 2f
CT244 t244 0 0.1f
M657 t244 nw83 vdd vdd pch w=2u l=180n
M658 t244 nw4 vdd vdd pch w=2u l=180n
CT245 t245 0 0.1f
M659 t244 nw83 t245 0 nch w=1u l=180n
M660 t245 nw4 0 0 nch w=1u l=180n
M661 nw86 t244 vdd vdd pch w=2u l=180n
M662 nw86 t244 0 0 nch w=1u l=180n
Cnw86 nw86 0 2f
CT246 t246 0 0.1f
M663 t246 nw84 vdd vdd pch w=2u l=180n
M664 t246 nw5 vdd vdd pch w=2u l=180n
CT247 t247 0 0.1f
M665 t246 nw84 t247 0 nch w=1u l=180n
M666 t247 nw5 0 0 nch w=1u l=180n
M667 nw87 t246 vdd vdd pch w=2u l=180n
M668 nw87 t246 0 0 nch w=1u l=180n
Cnw87 nw87 0 2f
CT248 t248 0 0.1f
M669 t248 nw78 vdd vdd pch w=2u l=180n
M670 t248 nw6 vdd vdd pch w=2u l=180n
CT249 t249 0 0.1f
M671 t248 nw78 t249 0 nch w=1u l=180n
M672 t249 nw6 0 0 nch w=1u l=180n
M673 nw88 t248 vdd vdd pch w=2u l=180n
M674 nw88 t248 0 0 nch w=1u l=180n
Cnw88 nw88 0 2f
CT250 t250 0 0.1f
M675 t250 nw85 0 0 nch w=1u l=180n
M676 t250 nw86 0 0 nch w=1u l=180n
M677 t250 nw87 0 0 nch w=1u l=180n
M678 t250 nw88 0 0 nch w=1u l=180n
CT251 t251 0 0.1f
M679 t251 nw85 vdd vdd pch w=2u l=180n
CT252 t252 0 0.1f
M680 t252 nw86 t251 vdd pch w=2u l=180n
CT253 t253 0 0.1f
M681 t253 nw87 t252 vdd pch w=2u l=180n
M682 t250 nw88 t253 vdd pch w=2u l=180n
M683 nw89 t250 vdd vdd pch w=2u l=180n
M684 nw89 t250 0 0 nch w=1u l=180n
Cnw89 nw89 0 2f
CT254 t254 0 0.1f
M685 t254 nw89 vdd vdd pch w=2u l=180n
M686 t254 nw89 0 0 nch w=1u l=180n
M687 ny5 t254 vdd vdd pch w=2u l=180n
M688 ny5 t254 0 0 nch w=1u l=180n
Cny5 ny5 0 2f
CT255 t255 0 0.1f
CT256 t256 0 0.1f
CT257 t257 0 0.1f
M689 t255 na6 vdd vdd pch w=2u l=180n
M690 t255 nb6 vdd vdd pch w=2u l=180n
CT258 t258 0 0.1f
M691 t255 na6 t258 0 nch w=1u l=180n
M692 t258 nb6 0 0 nch w=1u l=180n
M693 t256 na6 vdd vdd pch w=2u l=180n
M694 t256 t255 vdd vdd pch w=2u l=180n
CT259 t259 0 0.1f
M695 t256 na6 t259 0 nch w=1u l=180n
M696 t259 t255 0 0 nch w=1u l=180n
M697 t257 nb6 vdd vdd pch w=2u l=180n
M698 t257 t255 vdd vdd pch w=2u l=180n
CT260 t260 0 0.1f
M699 t257 nb6 t260 0 nch w=1u l=180n
M700 t260 t255 0 0 nch w=1u l=180n
M701 nw91 t256 vdd vdd pch w=2u l=180n
M702 nw91 t257 vdd vdd pch w=2u l=180n
CT261 t261 0 0.1f
M703 nw91 t256 t261 0 nch w=1u l=180n
M704 t261 t257 0 0 nch w=1u l=180n
Cnw91 nw91 0 2f
CT262 t262 0 0.1f
CT263 t263 0 0.1f
CT264 t264 0 0.1f
M705 t262 nw91 vdd vdd pch w=2u l=180n
M706 t262 nw81 vdd vdd pch w=2u l=180n
CT265 t265 0 0.1f
M707 t262 nw91 t265 0 nch w=1u l=180n
M708 t265 nw81 0 0 nch w=1u l=180n
M709 t263 nw91 vdd vdd pch w=2u l=180n
M710 t263 t262 vdd vdd pch w=2u l=180n
CT266 t266 0 0.1f
M711 t263 nw91 t266 0 nch w=1u l=180n
M712 t266 t262 0 0 nch w=1u l=180n
M713 t264 nw81 vdd vdd pch w=2u l=180n
M714 t264 t262 vdd vdd pch w=2u l=180n
CT267 t267 0 0.1f
M715 t264 nw81 t267 0 nch w=1u l=180n
M716 t267 t262 0 0 nch w=1u l=180n
M717 nw92 t263 vdd vdd pch w=2u l=180n
M718 nw92 t264 vdd vdd pch w=2u l=180n
CT268 t268 0 0.1f
M719 nw92 t263 t268 0 nch w=1u l=180n
M720 t268 t264 0 0 nch w=1u l=180n
Cnw92 nw92 0 2f
M721 nw93 na6 vdd vdd pch w=2u l=180n
M722 nw93 nb6 vdd vdd pch w=2u l=180n
CT269 t269 0 0.1f
M723 nw93 na6 t269 0 nch w=1u l=180n
M724 t269 nb6 0 0 nch w=1u l=180n
Cnw93 nw93 0 2f
M725 nw94 nw91 vdd vdd pch w=2u l=180n
M726 nw94 nw81 vdd vdd pch w=2u l=180n
CT270 t270 0 0.1f
M727 nw94 nw91 t270 0 nch w=1u l=180n
M728 t270 nw81 0 0 nch w=1u l=180n
Cnw94 nw94 0 2f
M729 nw95 nw93 vdd vdd pch w=2u l=180n
M730 nw95 nw94 vdd vdd pch w=2u l=180n
CT271 t271 0 0.1f
M731 nw95 nw93 t271 0 nch w=1u l=180n
M732 t271 nw94 0 0 nch w=1u l=180n
Cnw95 nw95 0 2f
CT272 t272 0 0.1f
M733 t272 na6 vdd vdd pch w=2u l=180n
M734 t272 nb6 vdd vdd pch w=2u l=180n
CT273 t273 0 0.1f
M735 t272 na6 t273 0 nch w=1u l=180n
M736 t273 nb6 0 0 nch w=1u l=180n
M737 nw96 t272 vdd vdd pch w=2u l=180n
M738 nw96 t272 0 0 nch w=1u l=180n
Cnw96 nw96 0 2f
CT274 t274 0 0.1f
M739 t274 na6 0 0 nch w=1u l=180n
M740 t274 nb6 0 0 nch w=1u l=180n
CT275 t275 0 0.1f
M741 t275 na6 vdd vdd pch w=2u l=180n
M742 t274 nb6 t275 vdd pch w=2u l=180n
M743 nw97 t274 vdd vdd pch w=2u l=180n
M744 nw97 t274 0 0 nch w=1u l=180n
Cnw97 nw97 0 2f
CT276 t276 0 0.1f
CT277 t277 0 0.1f
CT278 t278 0 0.1f
M745 t276 na6 vdd vdd pch w=2u l=180n
M746 t276 nb6 vdd vdd pch w=2u l=180n
CT279 t279 0 0.1f
M747 t276 na6 t279 0 nch w=1u l=180n
M748 t279 nb6 0 0 nch w=1u l=180n
M749 t277 na6 vdd vdd pch w=2u l=180n
M750 t277 t276 vdd vdd pch w=2u l=180n
CT280 t280 0 0.1f
M751 t277 na6 t280 0 nch w=1u l=180n
M752 t280 t276 0 0 nch w=1u l=180n
M753 t278 nb6 vdd vdd pch w=2u l=180n
M754 t278 t276 vdd vdd pch w=2u l=180n
CT281 t281 0 0.1f
M755 t278 nb6 t281 0 nch w=1u l=180n
M756 t281 t276 0 0 nch w=1u l=180n
M757 nw98 t277 vdd vdd pch w=2u l=180n
M758 nw98 t278 vdd vdd pch w=2u l=180n
CT282 t282 0 0.1f
M759 nw98 t277 t282 0 nch w=1u l=180n
M760 t282 t278 0 0 nch w=1u l=180n
Cnw98 nw98 0 2f
CT283 t283 0 0.1f
M761 t283 nw96 vdd vdd pch w=2u l=180n
M762 t283 nw3 vdd vdd pch w=2u l=180n
CT284 t284 0 0.1f
M763 t283 nw96 t284 0 nch w=1u l=180n
M764 t284 nw3 0 0 nch w=1u l=180n
M765 nw99 t283 vdd vdd pch w=2u l=180n
M766 nw99 t283 0 0 nch w=1u l=180n
Cnw99 nw99 0 2f
CT285 t285 0 0.1f
M767 t285 nw97 vdd vdd pch w=2u l=180n
M768 t285 nw4 vdd vdd pch w=2u l=180n
CT286 t286 0 0.1f
M769 t285 nw97 t286 0 nch w=1u l=180n
M770 t286 nw4 0 0 nch w=1u l=180n
M771 nw100 t285 vdd vdd pch w=2u l=180n
M772 nw100 t285 0 0 nch w=1u l=180n
Cnw100 nw100 0 2f
CT287 t287 0 0.1f
M773 t287 nw98 vdd vdd pch w=2u l=180n
M774 t287 nw5 vdd vdd pch w=2u l=180n
CT288 t288 0 0.1f
M775 t287 nw98 t288 0 nch w=1u l=180n
M776 t288 nw5 0 0 nch w=1u l=180n
M777 nw101 t287 vdd vdd pch w=2u l=180n
M778 nw101 t287 0 0 nch w=1u l=180n
Cnw101 nw101 0 2f
CT289 t289 0 0.1f
M779 t289 nw92 vdd vdd pch w=2u l=180n
M780 t289 nw6 vdd vdd pch w=2u l=180n
CT290 t290 0 0.1f
M781 t289 nw92 t290 0 nch w=1u l=180n
M782 t290 nw6 0 0 nch w=1u l=180n
M783 nw102 t289 vdd vdd pch w=2u l=180n
M784 nw102 t289 0 0 nch w=1u l=180n
Cnw102 nw102 0 2f
CT291 t291 0 0.1f
M785 t291 nw99 0 0 nch w=1u l=180n
M786 t291 nw100 0 0 nch w=1u l=180n
M787 t291 nw101 0 0 nch w=1u l=180n
M788 t291 nw102 0 0 nch w=1u l=180n
CT292 t292 0 0.1f
M789 t292 nw99 vdd vdd pch w=2u l=180n
CT293 t293 0 0.1f
M790 t293 nw100 t292 vdd pch w=2u l=180n
CT294 t294 0 0.1f
M791 t294 nw101 t293 vdd pch w=2u l=180n
M792 t291 nw102 t294 vdd pch w=2u l=180n
M793 nw103 t291 vdd vdd pch w=2u l=180n
M794 nw103 t291 0 0 nch w=1u l=180n
Cnw103 nw103 0 2f
CT295 t295 0 0.1f
M795 t295 nw103 vdd vdd pch w=2u l=180n
M796 t295 nw103 0 0 nch w=1u l=180n
M797 ny6 t295 vdd vdd pch w=2u l=180n
M798 ny6 t295 0 0 nch w=1u l=180n
Cny6 ny6 0 2f
CT296 t296 0 0.1f
CT297 t297 0 0.1f
CT298 t298 0 0.1f
M799 t296 na7 vdd vdd pch w=2u l=180n
M800 t296 nb7 vdd vdd pch w=2u l=180n
CT299 t299 0 0.1f
M801 t296 na7 t299 0 nch w=1u l=180n
M802 t299 nb7 0 0 nch w=1u l=180n
M803 t297 na7 vdd vdd pch w=2u l=180n
M804 t297 t296 vdd vdd pch w=2u l=180n
CT300 t300 0 0.1f
M805 t297 na7 t300 0 nch w=1u l=180n
M806 t300 t296 0 0 nch w=1u l=180n
M807 t298 nb7 vdd vdd pch w=2u l=180n
M808 t298 t296 vdd vdd pch w=2u l=180n
CT301 t301 0 0.1f
M809 t298 nb7 t301 0 nch w=1u l=180n
M810 t301 t296 0 0 nch w=1u l=180n
M811 nw105 t297 vdd vdd pch w=2u l=180n
M812 nw105 t298 vdd vdd pch w=2u l=180n
CT302 t302 0 0.1f
M813 nw105 t297 t302 0 nch w=1u l=180n
M814 t302 t298 0 0 nch w=1u l=180n
Cnw105 nw105 0 2f
CT303 t303 0 0.1f
CT304 t304 0 0.1f
CT305 t305 0 0.1f
M815 t303 nw105 vdd vdd pch w=2u l=180n
M816 t303 nw95 vdd vdd pch w=2u l=180n
CT306 t306 0 0.1f
M817 t303 nw105 t306 0 nch w=1u l=180n
M818 t306 nw95 0 0 nch w=1u l=180n
M819 t304 nw105 vdd vdd pch w=2u l=180n
M820 t304 t303 vdd vdd pch w=2u l=180n
CT307 t307 0 0.1f
M821 t304 nw105 t307 0 nch w=1u l=180n
M822 t307 t303 0 0 nch w=1u l=180n
M823 t305 nw95 vdd vdd pch w=2u l=180n
M824 t305 t303 vdd vdd pch w=2u l=180n
CT308 t308 0 0.1f
M825 t305 nw95 t308 0 nch w=1u l=180n
M826 t308 t303 0 0 nch w=1u l=180n
M827 nw106 t304 vdd vdd pch w=2u l=180n
M828 nw106 t305 vdd vdd pch w=2u l=180n
CT309 t309 0 0.1f
M829 nw106 t304 t309 0 nch w=1u l=180n
M830 t309 t305 0 0 nch w=1u l=180n
Cnw106 nw106 0 2f
M831 nw107 na7 vdd vdd pch w=2u l=180n
M832 nw107 nb7 vdd vdd pch w=2u l=180n
CT310 t310 0 0.1f
M833 nw107 na7 t310 0 nch w=1u l=180n
M834 t310 nb7 0 0 nch w=1u l=180n
Cnw107 nw107 0 2f
M835 nw108 nw105 vdd vdd pch w=2u l=180n
M836 nw108 nw95 vdd vdd pch w=2u l=180n
CT311 t311 0 0.1f
M837 nw108 nw105 t311 0 nch w=1u l=180n
M838 t311 nw95 0 0 nch w=1u l=180n
Cnw108 nw108 0 2f
M839 nw109 nw107 vdd vdd pch w=2u l=180n
M840 nw109 nw108 vdd vdd pch w=2u l=180n
CT312 t312 0 0.1f
M841 nw109 nw107 t312 0 nch w=1u l=180n
M842 t312 nw108 0 0 nch w=1u l=180n
Cnw109 nw109 0 2f
CT313 t313 0 0.1f
M843 t313 na7 vdd vdd pch w=2u l=180n
M844 t313 nb7 vdd vdd pch w=2u l=180n
CT314 t314 0 0.1f
M845 t313 na7 t314 0 nch w=1u l=180n
M846 t314 nb7 0 0 nch w=1u l=180n
M847 nw110 t313 vdd vdd pch w=2u l=180n
M848 nw110 t313 0 0 nch w=1u l=180n
Cnw110 nw110 0 2f
CT315 t315 0 0.1f
M849 t315 na7 0 0 nch w=1u l=180n
M850 t315 nb7 0 0 nch w=1u l=180n
CT316 t316 0 0.1f
M851 t316 na7 vdd vdd pch w=2u l=180n
M852 t315 nb7 t316 vdd pch w=2u l=180n
M853 nw111 t315 vdd vdd pch w=2u l=180n
M854 nw111 t315 0 0 nch w=1u l=180n
Cnw111 nw111 0 2f
CT317 t317 0 0.1f
CT318 t318 0 0.1f
CT319 t319 0 0.1f
M855 t317 na7 vdd vdd pch w=2u l=180n
M856 t317 nb7 vdd vdd pch w=2u l=180n
CT320 t320 0 0.1f
M857 t317 na7 t320 0 nch w=1u l=180n
M858 t320 nb7 0 0 nch w=1u l=180n
M859 t318 na7 vdd vdd pch w=2u l=180n
M860 t318 t317 vdd vdd pch w=2u l=180n
CT321 t321 0 0.1f
M861 t318 na7 t321 0 nch w=1u l=180n
M862 t321 t317 0 0 nch w=1u l=180n
M863 t319 nb7 vdd vdd pch w=2u l=180n
M864 t319 t317 vdd vdd pch w=2u l=180n
CT322 t322 0 0.1f
M865 t319 nb7 t322 0 nch w=1u l=180n
M866 t322 t317 0 0 nch w=1u l=180n
M867 nw112 t318 vdd vdd pch w=2u l=180n
M868 nw112 t319 vdd vdd pch w=2u l=180n
CT323 t323 0 0.1f
M869 nw112 t318 t323 0 nch w=1u l=180n
M870 t323 t319 0 0 nch w=1u l=180n
Cnw112 nw112 0 2f
CT324 t324 0 0.1f
M871 t324 nw110 vdd vdd pch w=2u l=180n
M872 t324 nw3 vdd vdd pch w=2u l=180n
CT325 t325 0 0.1f
M873 t324 nw110 t325 0 nch w=1u l=180n
M874 t325 nw3 0 0 nch w=1u l=180n
M875 nw113 t324 vdd vdd pch w=2u l=180n
M876 nw113 t324 0 0 nch w=1u l=180n
Cnw113 nw113 0 2f
CT326 t326 0 0.1f
M877 t326 nw111 vdd vdd pch w=2u l=180n
M878 t326 nw4 vdd vdd pch w=2u l=180n
CT327 t327 0 0.1f
M879 t326 nw111 t327 0 nch w=1u l=180n
M880 t327 nw4 0 0 nch w=1u l=180n
M881 nw114 t326 vdd vdd pch w=2u l=180n
M882 nw114 t326 0 0 nch w=1u l=180n
Cnw114 nw114 0 2f
CT328 t328 0 0.1f
M883 t328 nw112 vdd vdd pch w=2u l=180n
M884 t328 nw5 vdd vdd pch w=2u l=180n
CT329 t329 0 0.1f
M885 t328 nw112 t329 0 nch w=1u l=180n
M886 t329 nw5 0 0 nch w=1u l=180n
M887 nw115 t328 vdd vdd pch w=2u l=180n
M888 nw115 t328 0 0 nch w=1u l=180n
Cnw115 nw115 0 2f
CT330 t330 0 0.1f
M889 t330 nw106 vdd vdd pch w=2u l=180n
M890 t330 nw6 vdd vdd pch w=2u l=180n
CT331 t331 0 0.1f
M891 t330 nw106 t331 0 nch w=1u l=180n
M892 t331 nw6 0 0 nch w=1u l=180n
M893 nw116 t330 vdd vdd pch w=2u l=180n
M894 nw116 t330 0 0 nch w=1u l=180n
Cnw116 nw116 0 2f
CT332 t332 0 0.1f
M895 t332 nw113 0 0 nch w=1u l=180n
M896 t332 nw114 0 0 nch w=1u l=180n
M897 t332 nw115 0 0 nch w=1u l=180n
M898 t332 nw116 0 0 nch w=1u l=180n
CT333 t333 0 0.1f
M899 t333 nw113 vdd vdd pch w=2u l=180n
CT334 t334 0 0.1f
M900 t334 nw114 t333 vdd pch w=2u l=180n
CT335 t335 0 0.1f
M901 t335 nw115 t334 vdd pch w=2u l=180n
M902 t332 nw116 t335 vdd pch w=2u l=180n
M903 nw117 t332 vdd vdd pch w=2u l=180n
M904 nw117 t332 0 0 nch w=1u l=180n
Cnw117 nw117 0 2f
CT336 t336 0 0.1f
M905 t336 nw117 vdd vdd pch w=2u l=180n
M906 t336 nw117 0 0 nch w=1u l=180n
M907 ny7 t336 vdd vdd pch w=2u l=180n
M908 ny7 t336 0 0 nch w=1u l=180n
Cny7 ny7 0 2f
CT337 t337 0 0.1f
CT338 t338 0 0.1f
CT339 t339 0 0.1f
M909 t337 na8 vdd vdd pch w=2u l=180n
M910 t337 nb8 vdd vdd pch w=2u l=180n
CT340 t340 0 0.1f
M911 t337 na8 t340 0 nch w=1u l=180n
M912 t340 nb8 0 0 nch w=1u l=180n
M913 t338 na8 vdd vdd pch w=2u l=180n
M914 t338 t337 vdd vdd pch w=2u l=180n
CT341 t341 0 0.1f
M915 t338 na8 t341 0 nch w=1u l=180n
M916 t341 t337 0 0 nch w=1u l=180n
M917 t339 nb8 vdd vdd pch w=2u l=180n
M918 t339 t337 vdd vdd pch w=2u l=180n
CT342 t342 0 0.1f
M919 t339 nb8 t342 0 nch w=1u l=180n
M920 t342 t337 0 0 nch w=1u l=180n
M921 nw119 t338 vdd vdd pch w=2u l=180n
M922 nw119 t339 vdd vdd pch w=2u l=180n
CT343 t343 0 0.1f
M923 nw119 t338 t343 0 nch w=1u l=180n
M924 t343 t339 0 0 nch w=1u l=180n
Cnw119 nw119 0 2f
CT344 t344 0 0.1f
CT345 t345 0 0.1f
CT346 t346 0 0.1f
M925 t344 nw119 vdd vdd pch w=2u l=180n
M926 t344 nw109 vdd vdd pch w=2u l=180n
CT347 t347 0 0.1f
M927 t344 nw119 t347 0 nch w=1u l=180n
M928 t347 nw109 0 0 nch w=1u l=180n
M929 t345 nw119 vdd vdd pch w=2u l=180n
M930 t345 t344 vdd vdd pch w=2u l=180n
CT348 t348 0 0.1f
M931 t345 nw119 t348 0 nch w=1u l=180n
M932 t348 t344 0 0 nch w=1u l=180n
M933 t346 nw109 vdd vdd pch w=2u l=180n
M934 t346 t344 vdd vdd pch w=2u l=180n
CT349 t349 0 0.1f
M935 t346 nw109 t349 0 nch w=1u l=180n
M936 t349 t344 0 0 nch w=1u l=180n
M937 nw120 t345 vdd vdd pch w=2u l=180n
M938 nw120 t346 vdd vdd pch w=2u l=180n
CT350 t350 0 0.1f
M939 nw120 t345 t350 0 nch w=1u l=180n
M940 t350 t346 0 0 nch w=1u l=180n
Cnw120 nw120 0 2f
M941 nw121 na8 vdd vdd pch w=2u l=180n
M942 nw121 nb8 vdd vdd pch w=2u l=180n
CT351 t351 0 0.1f
M943 nw121 na8 t351 0 nch w=1u l=180n
M944 t351 nb8 0 0 nch w=1u l=180n
Cnw121 nw121 0 2f
M945 nw122 nw119 vdd vdd pch w=2u l=180n
M946 nw122 nw109 vdd vdd pch w=2u l=180n
CT352 t352 0 0.1f
M947 nw122 nw119 t352 0 nch w=1u l=180n
M948 t352 nw109 0 0 nch w=1u l=180n
Cnw122 nw122 0 2f
M949 nw123 nw121 vdd vdd pch w=2u l=180n
M950 nw123 nw122 vdd vdd pch w=2u l=180n
CT353 t353 0 0.1f
M951 nw123 nw121 t353 0 nch w=1u l=180n
M952 t353 nw122 0 0 nch w=1u l=180n
Cnw123 nw123 0 2f
CT354 t354 0 0.1f
M953 t354 na8 vdd vdd pch w=2u l=180n
M954 t354 nb8 vdd vdd pch w=2u l=180n
CT355 t355 0 0.1f
M955 t354 na8 t355 0 nch w=1u l=180n
M956 t355 nb8 0 0 nch w=1u l=180n
M957 nw124 t354 vdd vdd pch w=2u l=180n
M958 nw124 t354 0 0 nch w=1u l=180n
Cnw124 nw124 0 2f
CT356 t356 0 0.1f
M959 t356 na8 0 0 nch w=1u l=180n
M960 t356 nb8 0 0 nch w=1u l=180n
CT357 t357 0 0.1f
M961 t357 na8 vdd vdd pch w=2u l=180n
M962 t356 nb8 t357 vdd pch w=2u l=180n
M963 nw125 t356 vdd vdd pch w=2u l=180n
M964 nw125 t356 0 0 nch w=1u l=180n
Cnw125 nw125 0 2f
CT358 t358 0 0.1f
CT359 t359 0 0.1f
CT360 t360 0 0.1f
M965 t358 na8 vdd vdd pch w=2u l=180n
M966 t358 nb8 vdd vdd pch w=2u l=180n
CT361 t361 0 0.1f
M967 t358 na8 t361 0 nch w=1u l=180n
M968 t361 nb8 0 0 nch w=1u l=180n
M969 t359 na8 vdd vdd pch w=2u l=180n
M970 t359 t358 vdd vdd pch w=2u l=180n
CT362 t362 0 0.1f
M971 t359 na8 t362 0 nch w=1u l=180n
M972 t362 t358 0 0 nch w=1u l=180n
M973 t360 nb8 vdd vdd pch w=2u l=180n
M974 t360 t358 vdd vdd pch w=2u l=180n
CT363 t363 0 0.1f
M975 t360 nb8 t363 0 nch w=1u l=180n
M976 t363 t358 0 0 nch w=1u l=180n
M977 nw126 t359 vdd vdd pch w=2u l=180n
M978 nw126 t360 vdd vdd pch w=2u l=180n
CT364 t364 0 0.1f
M979 nw126 t359 t364 0 nch w=1u l=180n
M980 t364 t360 0 0 nch w=1u l=180n
Cnw126 nw126 0 2f
CT365 t365 0 0.1f
M981 t365 nw124 vdd vdd pch w=2u l=180n
M982 t365 nw3 vdd vdd pch w=2u l=180n
CT366 t366 0 0.1f
M983 t365 nw124 t366 0 nch w=1u l=180n
M984 t366 nw3 0 0 nch w=1u l=180n
M985 nw127 t365 vdd vdd pch w=2u l=180n
M986 nw127 t365 0 0 nch w=1u l=180n
Cnw127 nw127 0 2f
CT367 t367 0 0.1f
M987 t367 nw125 vdd vdd pch w=2u l=180n
M988 t367 nw4 vdd vdd pch w=2u l=180n
CT368 t368 0 0.1f
M989 t367 nw125 t368 0 nch w=1u l=180n
M990 t368 nw4 0 0 nch w=1u l=180n
M991 nw128 t367 vdd vdd pch w=2u l=180n
M992 nw128 t367 0 0 nch w=1u l=180n
Cnw128 nw128 0 2f
CT369 t369 0 0.1f
M993 t369 nw126 vdd vdd pch w=2u l=180n
M994 t369 nw5 vdd vdd pch w=2u l=180n
CT370 t370 0 0.1f
M995 t369 nw126 t370 0 nch w=1u l=180n
M996 t370 nw5 0 0 nch w=1u l=180n
M997 nw129 t369 vdd vdd pch w=2u l=180n
M998 nw129 t369 0 0 nch w=1u l=180n
Cnw129 nw129 0 2f
CT371 t371 0 0.1f
M999 t371 nw120 vdd vdd pch w=2u l=180n
M1000 t371 nw6 vdd vdd pch w=2u l=180n
CT372 t372 0 0.1f
M1001 t371 nw120 t372 0 nch w=1u l=180n
M1002 t372 nw6 0 0 nch w=1u l=180n
M1003 nw130 t371 vdd vdd pch w=2u l=180n
M1004 nw130 t371 0 0 nch w=1u l=180n
Cnw130 nw130 0 2f
CT373 t373 0 0.1f
M1005 t373 nw127 0 0 nch w=1u l=180n
M1006 t373 nw128 0 0 nch w=1u l=180n
M1007 t373 nw129 0 0 nch w=1u l=180n
M1008 t373 nw130 0 0 nch w=1u l=180n
CT374 t374 0 0.1f
M1009 t374 nw127 vdd vdd pch w=2u l=180n
CT375 t375 0 0.1f
M1010 t375 nw128 t374 vdd pch w=2u l=180n
CT376 t376 0 0.1f
M1011 t376 nw129 t375 vdd pch w=2u l=180n
M1012 t373 nw130 t376 vdd pch w=2u l=180n
M1013 nw131 t373 vdd vdd pch w=2u l=180n
M1014 nw131 t373 0 0 nch w=1u l=180n
Cnw131 nw131 0 2f
CT377 t377 0 0.1f
M1015 t377 nw131 vdd vdd pch w=2u l=180n
M1016 t377 nw131 0 0 nch w=1u l=180n
M1017 ny8 t377 vdd vdd pch w=2u l=180n
M1018 ny8 t377 0 0 nch w=1u l=180n
Cny8 ny8 0 2f
CT378 t378 0 0.1f
M1019 t378 ny0 0 0 nch w=1u l=180n
M1020 t378 ny1 0 0 nch w=1u l=180n
M1021 t378 ny2 0 0 nch w=1u l=180n
M1022 t378 ny3 0 0 nch w=1u l=180n
CT379 t379 0 0.1f
M1023 t379 ny0 vdd vdd pch w=2u l=180n
CT380 t380 0 0.1f
M1024 t380 ny1 t379 vdd pch w=2u l=180n
CT381 t381 0 0.1f
M1025 t381 ny2 t380 vdd pch w=2u l=180n
M1026 t378 ny3 t381 vdd pch w=2u l=180n
M1027 nw133 t378 vdd vdd pch w=2u l=180n
M1028 nw133 t378 0 0 nch w=1u l=180n
Cnw133 nw133 0 2f
CT382 t382 0 0.1f
M1029 t382 ny4 0 0 nch w=1u l=180n
M1030 t382 ny5 0 0 nch w=1u l=180n
M1031 t382 ny6 0 0 nch w=1u l=180n
M1032 t382 ny7 0 0 nch w=1u l=180n
CT383 t383 0 0.1f
M1033 t383 ny4 vdd vdd pch w=2u l=180n
CT384 t384 0 0.1f
M1034 t384 ny5 t383 vdd pch w=2u l=180n
CT385 t385 0 0.1f
M1035 t385 ny6 t384 vdd pch w=2u l=180n
M1036 t382 ny7 t385 vdd pch w=2u l=180n
M1037 nw134 t382 vdd vdd pch w=2u l=180n
M1038 nw134 t382 0 0 nch w=1u l=180n
Cnw134 nw134 0 2f
CT386 t386 0 0.1f
M1039 t386 nw133 0 0 nch w=1u l=180n
M1040 t386 nw134 0 0 nch w=1u l=180n
M1041 t386 ny8 0 0 nch w=1u l=180n
CT387 t387 0 0.1f
M1042 t387 nw133 vdd vdd pch w=2u l=180n
CT388 t388 0 0.1f
M1043 t388 nw134 t387 vdd pch w=2u l=180n
M1044 t386 ny8 t388 vdd pch w=2u l=180n
M1045 nw135 t386 vdd vdd pch w=2u l=180n
M1046 nw135 t386 0 0 nch w=1u l=180n
Cnw135 nw135 0 2f
M1047 nzero nw135 vdd vdd pch w=2u l=180n
M1048 nzero nw135 0 0 nch w=1u l=180n
Cnzero nzero 0 2f
CT389 t389 0 0.1f
M1049 t389 nw123 vdd vdd pch w=2u l=180n
M1050 t389 nw6 vdd vdd pch w=2u l=180n
CT390 t390 0 0.1f
M1051 t389 nw123 t390 0 nch w=1u l=180n
M1052 t390 nw6 0 0 nch w=1u l=180n
M1053 ncarry t389 vdd vdd pch w=2u l=180n
M1054 ncarry t389 0 0 nch w=1u l=180n
Cncarry ncarry 0 2f
.model nch NMOS (vto=0.45 kp=200u lambda=0.05)
.model pch PMOS (vto=-0.45 kp=100u lambda=0.05)
* outputs: ny0 ny1 ny2 ny3 ny4 ny5 ny6 ny7 ny8 nzero ncarry
.end
