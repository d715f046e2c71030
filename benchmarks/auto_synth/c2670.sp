* c2670 (c2670: 12-bit ALU and comparator): 156 gates, 1278 transistors
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
VIN9 na9 0 PULSE(0 1.8 2.56e-07 20p 20p 5.12e-07 1.024e-06)
VIN10 na10 0 PULSE(0 1.8 5.12e-07 20p 20p 1.024e-06 2.048e-06)
VIN11 na11 0 PULSE(0 1.8 1.024e-06 20p 20p 2.048e-06 4.096e-06)
VIN12 nb0 0 PULSE(0 1.8 2.048e-06 20p 20p 4.096e-06 8.192e-06)
VIN13 nb1 0 PULSE(0 1.8 4.096e-06 20p 20p 8.192e-06 1.6384e-05)
VIN14 nb2 0 PULSE(0 1.8 8.192e-06 20p 20p 1.6384e-05 3.2768e-05)
VIN15 nb3 0 PULSE(0 1.8 1.6384e-05 20p 20p 3.2768e-05 6.5536e-05)
VIN16 nb4 0 PULSE(0 1.8 3.2768e-05 20p 20p 6.5536e-05 0.000131072)
VIN17 nb5 0 PULSE(0 1.8 6.5536e-05 20p 20p 0.000131072 0.000262144)
VIN18 nb6 0 PULSE(0 1.8 0.000131072 20p 20p 0.000262144 0.000524288)
VIN19 nb7 0 PULSE(0 1.8 0.000262144 20p 20p 0.000524288 0.001048576)
VIN20 nb8 0 PULSE(0 1.8 0.000524288 20p 20p 0.001048576 0.002097152)
VIN21 nb9 0 PULSE(0 1.8 0.001048576 20p 20p 0.002097152 0.004194304)
VIN22 nb10 0 PULSE(0 1.8 0.002097152 20p 20p 0.004194304 0.008388608)
VIN23 nb11 0 PULSE(0 1.8 0.004194304 20p 20p 0.008388608 0.016777216)
VIN24 ncin 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
CT1 t1 0 0.1f
CT2 t2 0 0.1f
CT3 t3 0 0.1f
M1 t1 na0 vdd vdd pch w=2u l=180n
M2 t1 nb0 vdd vdd pch w=2u l=180n
CT4 t4 0 0.1f
M3 t1 na0 t4 0 nch w=1u l=180n
M4 t4 nb0 0 0 nch w=1u l=180n
M5 t2 na0 vdd vdd pch w=2u l=180n
M6 t2 t1 vdd vdd pch w=2u l=180n
CT5 t5 0 0.1f
M7 t2 na0 t5 0 nch w=1u l=180n
M8 t5 t1 0 0 nch w=1u l=180n
M9 t3 nb0 vdd vdd pch w=2u l=180n
M10 t3 t1 vdd vdd pch w=2u l=180n
CT6 t6 0 0.1f
M11 t3 nb0 t6 0 nch w=1u l=180n
M12 t6 t1 0 0 nch w=1u l=180n
M13 nw1 t2 vdd vdd pch w=2u l=180n
M14 nw1 t3 vdd vdd pch w=2u l=180n
CT7 t7 0 0.1f
M15 nw1 t2 t7 0 nch w=1u l=180n
M16 t7 t3 0 0 nch w=1u l=180n
Cnw1 nw1 0 2f
CT8 t8 0 0.1f
CT9 t9 0 0.1f
CT10 t10 0 0.1f
M17 t8 nw1 vdd vdd pch w=2u l=180n
M18 t8 ncin vdd vdd pch w=2u l=180n
CT11 t11 0 0.1f
M19 t8 nw1 t11 0 nch w=1u l=180n
M20 t11 ncin 0 0 nch w=1u l=180n
M21 t9 nw1 vdd vdd pch w=2u l=180n
M22 t9 t8 vdd vdd pch w=2u l=180n
CT12 t12 0 0.1f
M23 t9 nw1 t12 0 nch w=1u l=180n
M24 t12 t8 0 0 nch w=1u l=180n
M25 t10 ncin vdd vdd pch w=2u l=180n
M26 t10 t8 vdd vdd pch w=2u l=180n
CT13 t13 0 0.1f
M27 t10 ncin t13 0 nch w=1u l=180n
M28 t13 t8 0 0 nch w=1u l=180n
M29 nw2 t9 vdd vdd pch w=2u l=180n
M30 nw2 t10 vdd vdd pch w=2u l=180n
CT14 t14 0 0.1f
M31 nw2 t9 t14 0 nch w=1u l=180n
M32 t14 t10 0 0 nch w=1u l=180n
Cnw2 nw2 0 2f
M33 nw3 na0 vdd vdd pch w=2u l=180n
M34 nw3 nb0 vdd vdd pch w=2u l=180n
CT15 t15 0 0.1f
M35 nw3 na0 t15 0 nch w=1u l=180n
M36 t15 nb0 0 0 nch w=1u l=180n
Cnw3 nw3 0 2f
M37 nw4 nw1 vdd vdd pch w=2u l=180n
M38 nw4 ncin vdd vdd pch w=2u l=180n
CT16 t16 0 0.1f
M39 nw4 nw1 t16 0 nch w=1u l=180n
M40 t16 ncin 0 0 nch w=1u l=180n
Cnw4 nw4 0 2f
M41 nw5 nw3 vdd vdd pch w=2u l=180n
M42 nw5 nw4 vdd vdd pch w=2u l=180n
CT17 t17 0 0.1f
M43 nw5 nw3 t17 0 nch w=1u l=180n
M44 t17 nw4 0 0 nch w=1u l=180n
Cnw5 nw5 0 2f
CT18 t18 0 0.1f
M45 t18 nw2 vdd vdd pch w=2u l=180n
M46 t18 nw2 0 0 nch w=1u l=180n
M47 ns0 t18 vdd vdd pch w=2u l=180n
M48 ns0 t18 0 0 nch w=1u l=180n
Cns0 ns0 0 2f
CT19 t19 0 0.1f
CT20 t20 0 0.1f
CT21 t21 0 0.1f
M49 t19 na1 vdd vdd pch w=2u l=180n
M50 t19 nb1 vdd vdd pch w=2u l=180n
CT22 t22 0 0.1f
M51 t19 na1 t22 0 nch w=1u l=180n
M52 t22 nb1 0 0 nch w=1u l=180n
M53 t20 na1 vdd vdd pch w=2u l=180n
M54 t20 t19 vdd vdd pch w=2u l=180n
CT23 t23 0 0.1f
M55 t20 na1 t23 0 nch w=1u l=180n
M56 t23 t19 0 0 nch w=1u l=180n
M57 t21 nb1 vdd vdd pch w=2u l=180n
M58 t21 t19 vdd vdd pch w=2u l=180n
CT24 t24 0 0.1f
M59 t21 nb1 t24 0 nch w=1u l=180n
M60 t24 t19 0 0 nch w=1u l=180n
M61 nw7 t20 vdd vdd pch w=2u l=180n
M62 nw7 t21 vdd vdd pch w=2u l=180n
CT25 t25 0 0.1f
M63 nw7 t20 t25 0 nch w=1u l=180n
M64 t25 t21 0 0 nch w=1u l=180n
Cnw7 nw7 0 2f
CT26 t26 0 0.1f
CT27 t27 0 0.1f
CT28 t28 0 0.1f
M65 t26 nw7 vdd vdd pch w=2u l=180n
M66 t26 nw5 vdd vdd pch w=2u l=180n
CT29 t29 0 0.1f
M67 t26 nw7 t29 0 nch w=1u l=180n
M68 t29 nw5 0 0 nch w=1u l=180n
M69 t27 nw7 vdd vdd pch w=2u l=180n
M70 t27 t26 vdd vdd pch w=2u l=180n
CT30 t30 0 0.1f
M71 t27 nw7 t30 0 nch w=1u l=180n
M72 t30 t26 0 0 nch w=1u l=180n
M73 t28 nw5 vdd vdd pch w=2u l=180n
M74 t28 t26 vdd vdd pch w=2u l=180n
CT31 t31 0 0.1f
M75 t28 nw5 t31 0 nch w=1u l=180n
M76 t31 t26 0 0 nch w=1u l=180n
M77 nw8 t27 vdd vdd pch w=2u l=180n
M78 nw8 t28 vdd vdd pch w=2u l=180n
CT32 t32 0 0.1f
M79 nw8 t27 t32 0 nch w=1u l=180n
M80 t32 t28 0 0 nch w=1u l=180n
Cnw8 nw8 0 2f
M81 nw9 na1 vdd vdd pch w=2u l=180n
M82 nw9 nb1 vdd vdd pch w=2u l=180n
CT33 t33 0 0.1f
M83 nw9 na1 t33 0 nch w=1u l=180n
M84 t33 nb1 0 0 nch w=1u l=180n
Cnw9 nw9 0 2f
M85 nw10 nw7 vdd vdd pch w=2u l=180n
M86 nw10 nw5 vdd vdd pch w=2u l=180n
CT34 t34 0 0.1f
M87 nw10 nw7 t34 0 nch w=1u l=180n
M88 t34 nw5 0 0 nch w=1u l=180n
Cnw10 nw10 0 2f
M89 nw11 nw9 vdd vdd pch w=2u l=180n
M90 nw11 nw10 vdd vdd pch w=2u l=180n
CT35 t35 0 0.1f
M91 nw11 nw9 t35 0 nch w=1u l=180n
M92 t35 nw10 0 0 nch w=1u l=180n
Cnw11 nw11 0 2f
CT36 t36 0 0.1f
M93 t36 nw8 vdd vdd pch w=2u l=180n
M94 t36 nw8 0 0 nch w=1u l=180n
M95 ns1 t36 vdd vdd pch w=2u l=180n
M96 ns1 t36 0 0 nch w=1u l=180n
Cns1 ns1 0 2f
CT37 t37 0 0.1f
CT38 t38 0 0.1f
CT39 t39 0 0.1f
M97 t37 nw2 vdd vdd pch w=2u l=180n
M98 t37 nw8 vdd vdd pch w=2u l=180n
CT40 t40 0 0.1f
M99 t37 nw2 t40 0 nch w=1u l=180n
M100 t40 nw8 0 0 nch w=1u l=180n
M101 t38 nw2 vdd vdd pch w=2u l=180n
M102 t38 t37 vdd vdd pch w=2u l=180n
CT41 t41 0 0.1f
M103 t38 nw2 t41 0 nch w=1u l=180n
M104 t41 t37 0 0 nch w=1u l=180n
M105 t39 nw8 vdd vdd pch w=2u l=180n
M106 t39 t37 vdd vdd pch w=2u l=180n
CT42 t42 0 0.1f
M107 t39 nw8 t42 0 nch w=1u l=180n
M108 t42 t37 0 0 nch w=1u l=180n
M109 nw13 t38 vdd vdd pch w=2u l=180n
M110 nw13 t39 vdd vdd pch w=2u l=180n
CT43 t43 0 0.1f
M111 nw13 t38 t43 0 nch w=1u l=180n
M112 t43 t39 0 0 nch w=1u l=180n
Cnw13 nw13 0 2f
CT44 t44 0 0.1f
CT45 t45 0 0.1f
CT46 t46 0 0.1f
M113 t44 na2 vdd vdd pch w=2u l=180n
M114 t44 nb2 vdd vdd pch w=2u l=180n
CT47 t47 0 0.1f
M115 t44 na2 t47 0 nch w=1u l=180n
M116 t47 nb2 0 0 nch w=1u l=180n
M117 t45 na2 vdd vdd pch w=2u l=180n
M118 t45 t44 vdd vdd pch w=2u l=180n
CT48 t48 0 0.1f
M119 t45 na2 t48 0 nch w=1u l=180n
M120 t48 t44 0 0 nch w=1u l=180n
M121 t46 nb2 vdd vdd pch w=2u l=180n
M122 t46 t44 vdd vdd pch w=2u l=180n
CT49 t49 0 0.1f
M123 t46 nb2 t49 0 nch w=1u l=180n
M124 t49 t44 0 0 nch w=1u l=180n
M125 nw14 t45 vdd vdd pch w=2u l=180n
M126 nw14 t46 vdd vdd pch w=2u l=180n
CT50 t50 0 0.1f
M127 nw14 t45 t50 0 nch w=1u l=180n
M128 t50 t46 0 0 nch w=1u l=180n
Cnw14 nw14 0 2f
CT51 t51 0 0.1f
CT52 t52 0 0.1f
CT53 t53 0 0.1f
M129 t51 nw14 vdd vdd pch w=2u l=180n
M130 t51 nw11 vdd vdd pch w=2u l=180n
CT54 t54 0 0.1f
M131 t51 nw14 t54 0 nch w=1u l=180n
M132 t54 nw11 0 0 nch w=1u l=180n
M133 t52 nw14 vdd vdd pch w=2u l=180n
M134 t52 t51 vdd vdd pch w=2u l=180n
CT55 t55 0 0.1f
M135 t52 nw14 t55 0 nch w=1u l=180n
M136 t55 t51 0 0 nch w=1u l=180n
M137 t53 nw11 vdd vdd pch w=2u l=180n
M138 t53 t51 vdd vdd pch w=2u l=180n
CT56 t56 0 0.1f
M139 t53 nw11 t56 0 nch w=1u l=180n
M140 t56 t51 0 0 nch w=1u l=180n
M141 nw15 t52 vdd vdd pch w=2u l=180n
M142 nw15 t53 vdd vdd pch w=2u l=180n
CT57 t57 0 0.1f
M143 nw15 t52 t57 0 nch w=1u l=180n
M144 t57 t53 0 0 nch w=1u l=180n
Cnw15 nw15 0 2f
M145 nw16 na2 vdd vdd pch w=2u l=180n
M146 nw16 nb2 vdd vdd pch w=2u l=180n
CT58 t58 0 0.1f
M147 nw16 na2 t58 0 nch w=1u l=180n
M148 t58 nb2 0 0 nch w=1u l=180n
Cnw16 nw16 0 2f
M149 nw17 nw14 vdd vdd pch w=2u l=180n
M150 nw17 nw11 vdd vdd pch w=2u l=180n
CT59 t59 0 0.1f
M151 nw17 nw14 t59 0 nch w=1u l=180n
M152 t59 nw11 0 0 nch w=1u l=180n
Cnw17 nw17 0 2f
M153 nw18 nw16 vdd vdd pch w=2u l=180n
M154 nw18 nw17 vdd vdd pch w=2u l=180n
CT60 t60 0 0.1f
M155 nw18 nw16 t60 0 nch w=1u l=180n
M156 t60 nw17 0 0 nch w=1u l=180n
Cnw18 nw18 0 2f
CT61 t61 0 0.1f
M157 t61 nw15 vdd vdd pch w=2u l=180n
M158 t61 nw15 0 0 nch w=1u l=180n
M159 ns2 t61 vdd vdd pch w=2u l=180n
M160 ns2 t61 0 0 nch w=1u l=180n
Cns2 ns2 0 2f
CT62 t62 0 0.1f
CT63 t63 0 0.1f
CT64 t64 0 0.1f
M161 t62 nw13 vdd vdd pch w=2u l=180n
M162 t62 nw15 vdd vdd pch w=2u l=180n
CT65 t65 0 0.1f
M163 t62 nw13 t65 0 nch w=1u l=180n
M164 t65 nw15 0 0 nch w=1u l=180n
M165 t63 nw13 vdd vdd pch w=2u l=180n
M166 t63 t62 vdd vdd pch w=2u l=180n
CT66 t66 0 0.1f
M167 t63 nw13 t66 0 nch w=1u l=180n
M168 t66 t62 0 0 nch w=1u l=180n
M169 t64 nw15 vdd vdd pch w=2u l=180n
M170 t64 t62 vdd vdd pch w=2u l=180n
CT67 t67 0 0.1f
M171 t64 nw15 t67 0 nch w=1u l=180n
M172 t67 t62 0 0 nch w=1u l=180n
M173 nw20 t63 vdd vdd pch w=2u l=180n
M174 nw20 t64 vdd vdd pch w=2u l=180n
CT68 t68 0 0.1f
M175 nw20 t63 t68 0 nch w=1u l=180n
M176 t68 t64 0 0 nch w=1u l=180n
Cnw20 nw20 0 2f
CT69 t69 0 0.1f
CT70 t70 0 0.1f
CT71 t71 0 0.1f
M177 t69 na3 vdd vdd pch w=2u l=180n
M178 t69 nb3 vdd vdd pch w=2u l=180n
CT72 t72 0 0.1f
M179 t69 na3 t72 0 nch w=1u l=180n
M180 t72 nb3 0 0 nch w=1u l=180n
M181 t70 na3 vdd vdd pch w=2u l=180n
M182 t70 t69 vdd vdd pch w=2u l=180n
CT73 t73 0 0.1f
M183 t70 na3 t73 0 nch w=1u l=180n
M184 t73 t69 0 0 nch w=1u l=180n
M185 t71 nb3 vdd vdd pch w=2u l=180n
M186 t71 t69 vdd vdd pch w=2u l=180n
CT74 t74 0 0.1f
M187 t71 nb3 t74 0 nch w=1u l=180n
M188 t74 t69 0 0 nch w=1u l=180n
M189 nw21 t70 vdd vdd pch w=2u l=180n
M190 nw21 t71 vdd vdd pch w=2u l=180n
CT75 t75 0 0.1f
M191 nw21 t70 t75 0 nch w=1u l=180n
M192 t75 t71 0 0 nch w=1u l=180n
Cnw21 nw21 0 2f
CT76 t76 0 0.1f
CT77 t77 0 0.1f
CT78 t78 0 0.1f
M193 t76 nw21 vdd vdd pch w=2u l=180n
M194 t76 nw18 vdd vdd pch w=2u l=180n
CT79 t79 0 0.1f
M195 t76 nw21 t79 0 nch w=1u l=180n
M196 t79 nw18 0 0 nch w=1u l=180n
M197 t77 nw21 vdd vdd pch w=2u l=180n
M198 t77 t76 vdd vdd pch w=2u l=180n
CT80 t80 0 0.1f
M199 t77 nw21 t80 0 nch w=1u l=180n
M200 t80 t76 0 0 nch w=1u l=180n
M201 t78 nw18 vdd vdd pch w=2u l=180n
M202 t78 t76 vdd vdd pch w=2u l=180n
CT81 t81 0 0.1f
M203 t78 nw18 t81 0 nch w=1u l=180n
M204 t81 t76 0 0 nch w=1u l=180n
M205 nw22 t77 vdd vdd pch w=2u l=180n
M206 nw22 t78 vdd vdd pch w=2u l=180n
CT82 t82 0 0.1f
M207 nw22 t77 t82 0 nch w=1u l=180n
M208 t82 t78 0 0 nch w=1u l=180n
Cnw22 nw22 0 2f
M209 nw23 na3 vdd vdd pch w=2u l=180n
M210 nw23 nb3 vdd vdd pch w=2u l=180n
CT83 t83 0 0.1f
M211 nw23 na3 t83 0 nch w=1u l=180n
M212 t83 nb3 0 0 nch w=1u l=180n
Cnw23 nw23 0 2f
M213 nw24 nw21 vdd vdd pch w=2u l=180n
M214 nw24 nw18 vdd vdd pch w=2u l=180n
CT84 t84 0 0.1f
M215 nw24 nw21 t84 0 nch w=1u l=180n
M216 t84 nw18 0 0 nch w=1u l=180n
Cnw24 nw24 0 2f
M217 nw25 nw23 vdd vdd pch w=2u l=180n
M218 nw25 nw24 vdd vdd pch w=2u l=180n
CT85 t85 0 0.1f
M219 nw25 nw23 t85 0 nch w=1u l=180n
M220 t85 nw24 0 0 nch w=1u l=180n
Cnw25 nw25 0 2f
CT86 t86 0 0.1f
M221 t86 nw22 vdd vdd pch w=2u l=180n
M222 t86 nw22 0 0 nch w=1u l=180n
M223 ns3 t86 vdd vdd pch w=2u l=180n
M224 ns3 t86 0 0 nch w=1u l=180n
Cns3 ns3 0 2f
CT87 t87 0 0.1f
CT88 t88 0 0.1f
CT89 t89 0 0.1f
M225 t87 nw20 vdd vdd pch w=2u l=180n
M226 t87 nw22 vdd vdd pch w=2u l=180n
CT90 t90 0 0.1f
M227 t87 nw20 t90 0 nch w=1u l=180n
M228 t90 nw22 0 0 nch w=1u l=180n
M229 t88 nw20 vdd vdd pch w=2u l=180n
M230 t88 t87 vdd vdd pch w=2u l=180n
CT91 t91 0 0.1f
M231 t88 nw20 t91 0 nch w=1u l=180n
M232 t91 t87 0 0 nch w=1u l=180n
M233 t89 nw22 vdd vdd pch w=2u l=180n
M234 t89 t87 vdd vdd pch w=2u l=180n
CT92 t92 0 0.1f
M235 t89 nw22 t92 0 nch w=1u l=180n
M236 t92 t87 0 0 nch w=1u l=180n
M237 nw27 t88 vdd vdd pch w=2u l=180n
M238 nw27 t89 vdd vdd pch w=2u l=180n
CT93 t93 0 0.1f
M239 nw27 t88 t93 0 nch w=1u l=180n
M240 t93 t89 0 0 nch w=1u l=180n
Cnw27 nw27 0 2f
CT94 t94 0 0.1f
CT95 t95 0 0.1f
CT96 t96 0 0.1f
M241 t94 na4 vdd vdd pch w=2u l=180n
M242 t94 nb4 vdd vdd pch w=2u l=180n
CT97 t97 0 0.1f
M243 t94 na4 t97 0 nch w=1u l=180n
M244 t97 nb4 0 0 nch w=1u l=180n
M245 t95 na4 vdd vdd pch w=2u l=180n
M246 t95 t94 vdd vdd pch w=2u l=180n
CT98 t98 0 0.1f
M247 t95 na4 t98 0 nch w=1u l=180n
M248 t98 t94 0 0 nch w=1u l=180n
M249 t96 nb4 vdd vdd pch w=2u l=180n
M250 t96 t94 vdd vdd pch w=2u l=180n
CT99 t99 0 0.1f
M251 t96 nb4 t99 0 nch w=1u l=180n
M252 t99 t94 0 0 nch w=1u l=180n
M253 nw28 t95 vdd vdd pch w=2u l=180n
M254 nw28 t96 vdd vdd pch w=2u l=180n
CT100 t100 0 0.1f
M255 nw28 t95 t100 0 nch w=1u l=180n
M256 t100 t96 0 0 nch w=1u l=180n
Cnw28 nw28 0 2f
CT101 t101 0 0.1f
CT102 t102 0 0.1f
CT103 t103 0 0.1f
M257 t101 nw28 vdd vdd pch w=2u l=180n
M258 t101 nw25 vdd vdd pch w=2u l=180n
CT104 t104 0 0.1f
M259 t101 nw28 t104 0 nch w=1u l=180n
M260 t104 nw25 0 0 nch w=1u l=180n
M261 t102 nw28 vdd vdd pch w=2u l=180n
M262 t102 t101 vdd vdd pch w=2u l=180n
CT105 t105 0 0.1f
M263 t102 nw28 t105 0 nch w=1u l=180n
M264 t105 t101 0 0 nch w=1u l=180n
M265 t103 nw25 vdd vdd pch w=2u l=180n
M266 t103 t101 vdd vdd pch w=2u l=180n
CT106 t106 0 0.1f
M267 t103 nw25 t106 0 nch w=1u l=180n
M268 t106 t101 0 0 nch w=1u l=180n
M269 nw29 t102 vdd vdd pch w=2u l=180n
M270 nw29 t103 vdd vdd pch w=2u l=180n
CT107 t107 0 0.1f
M271 nw29 t102 t107 0 nch w=1u l=180n
M272 t107 t103 0 0 nch w=1u l=180n
Cnw29 nw29 0 2f
M273 nw30 na4 vdd vdd pch w=2u l=180n
M274 nw30 nb4 vdd vdd pch w=2u l=180n
CT108 t108 0 0.1f
M275 nw30 na4 t108 0 nch w=1u l=180n
M276 t108 nb4 0 0 nch w=1u l=180n
Cnw30 nw30 0 2f
M277 nw31 nw28 vdd vdd pch w=2u l=180n
M278 nw31 nw25 vdd vdd pch w=2u l=180n
CT109 t109 0 0.1f
M279 nw31 nw28 t109 0 nch w=1u l=180n
M280 t109 nw25 0 0 nch w=1u l=180n
Cnw31 nw31 0 2f
M281 nw32 nw30 vdd vdd pch w=2u l=180n
M282 nw32 nw31 vdd vdd pch w=2u l=180n
CT110 t110 0 0.1f
M283 nw32 nw30 t110 0 nch w=1u l=180n
M284 t110 nw31 0 0 nch w=1u l=180n
Cnw32 nw32 0 2f
CT111 t111 0 0.1f
M285 t111 nw29 vdd vdd pch w=2u l=180n
M286 t111 nw29 0 0 nch w=1u l=180n
M287 ns4 t111 vdd vdd pch w=2u l=180n
M288 ns4 t111 0 0 nch w=1u l=180n
Cns4 ns4 0 2f
CT112 t112 0 0.1f
CT113 t113 0 0.1f
CT114 t114 0 0.1f
M289 t112 nw27 vdd vdd pch w=2u l=180n
M290 t112 nw29 vdd vdd pch w=2u l=180n
CT115 t115 0 0.1f
M291 t112 nw27 t115 0 nch w=1u l=180n
M292 t115 nw29 0 0 nch w=1u l=180n
M293 t113 nw27 vdd vdd pch w=2u l=180n
M294 t113 t112 vdd vdd pch w=2u l=180n
CT116 t116 0 0.1f
M295 t113 nw27 t116 0 nch w=1u l=180n
M296 t116 t112 0 0 nch w=1u l=180n
M297 t114 nw29 vdd vdd pch w=2u l=180n
M298 t114 t112 vdd vdd pch w=2u l=180n
CT117 t117 0 0.1f
M299 t114 nw29 t117 0 nch w=1u l=180n
M300 t117 t112 0 0 nch w=1u l=180n
M301 nw34 t113 vdd vdd pch w=2u l=180n
M302 nw34 t114 vdd vdd pch w=2u l=180n
CT118 t118 0 0.1f
M303 nw34 t113 t118 0 nch w=1u l=180n
M304 t118 t114 0 0 nch w=1u l=180n
Cnw34 nw34 0 2f
CT119 t119 0 0.1f
CT120 t120 0 0.1f
CT121 t121 0 0.1f
M305 t119 na5 vdd vdd pch w=2u l=180n
M306 t119 nb5 vdd vdd pch w=2u l=180n
CT122 t122 0 0.1f
M307 t119 na5 t122 0 nch w=1u l=180n
M308 t122 nb5 0 0 nch w=1u l=180n
M309 t120 na5 vdd vdd pch w=2u l=180n
M310 t120 t119 vdd vdd pch w=2u l=180n
CT123 t123 0 0.1f
M311 t120 na5 t123 0 nch w=1u l=180n
M312 t123 t119 0 0 nch w=1u l=180n
M313 t121 nb5 vdd vdd pch w=2u l=180n
M314 t121 t119 vdd vdd pch w=2u l=180n
CT124 t124 0 0.1f
M315 t121 nb5 t124 0 nch w=1u l=180n
M316 t124 t119 0 0 nch w=1u l=180n
M317 nw35 t120 vdd vdd pch w=2u l=180n
M318 nw35 t121 vdd vdd pch w=2u l=180n
CT125 t125 0 0.1f
M319 nw35 t120 t125 0 nch w=1u l=180n
M320 t125 t121 0 0 nch w=1u l=180n
Cnw35 nw35 0 2f
CT126 t126 0 0.1f
CT127 t127 0 0.1f
CT128 t128 0 0.1f
M321 t126 nw35 vdd vdd pch w=2u l=180n
M322 t126 nw32 vdd vdd pch w=2u l=180n
CT129 t129 0 0.1f
M323 t126 nw35 t129 0 nch w=1u l=180n
M324 t129 nw32 0 0 nch w=1u l=180n
M325 t127 nw35 vdd vdd pch w=2u l=180n
M326 t127 t126 vdd vdd pch w=2u l=180n
CT130 t130 0 0.1f
M327 t127 nw35 t130 0 nch w=1u l=180n
M328 t130 t126 0 0 nch w=1u l=180n
M329 t128 nw32 vdd vdd pch w=2u l=180n
M330 t128 t126 vdd vdd pch w=2u l=180n
CT131 t131 0 0.1f
M331 t128 nw32 t131 0 nch w=1u l=180n
M332 t131 t126 0 0 nch w=1u l=180n
M333 nw36 t127 vdd vdd pch w=2u l=180n
M334 nw36 t128 vdd vdd pch w=2u l=180n
CT132 t132 0 0.1f
M335 nw36 t127 t132 0 nch w=1u l=180n
M336 t132 t128 0 0 nch w=1u l=180n
Cnw36 nw36 0 2f
M337 nw37 na5 vdd vdd pch w=2u l=180n
M338 nw37 nb5 vdd vdd pch w=2u l=180n
CT133 t133 0 0.1f
M339 nw37 na5 t133 0 nch w=1u l=180n
M340 t133 nb5 0 0 nch w=1u l=180n
Cnw37 nw37 0 2f
M341 nw38 nw35 vdd vdd pch w=2u l=180n
M342 nw38 nw32 vdd vdd pch w=2u l=180n
CT134 t134 0 0.1f
M343 nw38 nw35 t134 0 nch w=1u l=180n
M344 t134 nw32 0 0 nch w=1u l=180n
Cnw38 nw38 0 2f
M345 nw39 nw37 vdd vdd pch w=2u l=180n
M346 nw39 nw38 vdd vdd pch w=2u l=180n
CT135 t135 0 0.1f
M347 nw39 nw37 t135 0 nch w=1u l=180n
M348 t135 nw38 0 0 nch w=1u l=180n
Cnw39 nw39 0 2f
CT136 t136 0 0.1f
M349 t136 nw36 vdd vdd pch w=2u l=180n
M350 t136 nw36 0 0 nch w=1u l=180n
M351 ns5 t136 vdd vdd pch w=2u l=180n
M352 ns5 t136 0 0 nch w=1u l=180n
Cns5 ns5 0 2f
CT137 t137 0 0.1f
CT138 t138 0 0.1f
CT139 t139 0 0.1f
M353 t137 nw34 vdd vdd pch w=2u l=180n
M354 t137 nw36 vdd vdd pch w=2u l=180n
CT140 t140 0 0.1f
M355 t137 nw34 t140 0 nch w=1u l=180n
M356 t140 nw36 0 0 nch w=1u l=180n
M357 t138 nw34 vdd vdd pch w=2u l=180n
M358 t138 t137 vdd vdd pch w=2u l=180n
CT141 t141 0 0.1f
M359 t138 nw34 t141 0 nch w=1u l=180n
M360 t141 t137 0 0 nch w=1u l=180n
M361 t139 nw36 vdd vdd pch w=2u l=180n
M362 t139 t137 vdd vdd pch w=2u l=180n
CT142 t142 0 0.1f
M363 t139 nw36 t142 0 nch w=1u l=180n
M364 t142 t137 0 0 nch w=1u l=180n
M365 nw41 t138 vdd vdd pch w=2u l=180n
M366 nw41 t139 vdd vdd pch w=2u l=180n
CT143 t143 0 0.1f
M367 nw41 t138 t143 0 nch w=1u l=180n
M368 t143 t139 0 0 nch w=1u l=180n
Cnw41 nw41 0 2f
CT144 t144 0 0.1f
CT145 t145 0 0.1f
CT146 t146 0 0.1f
M369 t144 na6 vdd vdd pch w=2u l=180n
M370 t144 nb6 vdd vdd pch w=2u l=180n
CT147 t147 0 0.1f
M371 t144 na6 t147 0 nch w=1u l=180n
M372 t147 nb6 0 0 nch w=1u l=180n
M373 t145 na6 vdd vdd pch w=2u l=180n
M374 t145 t144 vdd vdd pch w=2u l=180n
CT148 t148 0 0.1f
M375 t145 na6 t148 0 nch w=1u l=180n
M376 t148 t144 0 0 nch w=1u l=180n
M377 t146 nb6 vdd vdd pch w=2u l=180n
M378 t146 t144 vdd vdd pch w=2u l=180n
CT149 t149 0 0.1f
M379 t146 nb6 t149 0 nch w=1u l=180n
M380 t149 t144 0 0 nch w=1u l=180n
M381 nw42 t145 vdd vdd pch w=2u l=180n
M382 nw42 t146 vdd vdd pch w=2u l=180n
CT150 t150 0 0.1f
M383 nw42 t145 t150 0 nch w=1u l=180n
M384 t150 t146 0 0 nch w=1u l=180n
Cnw42 nw42 0 2f
CT151 t151 0 0.1f
CT152 t152 0 0.1f
CT153 t153 0 0.1f
M385 t151 nw42 vdd vdd pch w=2u l=180n
M386 t151 nw39 vdd vdd pch w=2u l=180n
CT154 t154 0 0.1f
M387 t151 nw42 t154 0 nch w=1u l=180n
M388 t154 nw39 0 0 nch w=1u l=180n
M389 t152 nw42 vdd vdd pch w=2u l=180n
M390 t152 t151 vdd vdd pch w=2u l=180n
CT155 t155 0 0.1f
M391 t152 nw42 t155 0 nch w=1u l=180n
M392 t155 t151 0 0 nch w=1u l=180n
M393 t153 nw39 vdd vdd pch w=2u l=180n
M394 t153 t151 vdd vdd pch w=2u l=180n
CT156 t156 0 0.1f
M395 t153 nw39 t156 0 nch w=1u l=180n
M396 t156 t151 0 0 nch w=1u l=180n
M397 nw43 t152 vdd vdd pch w=2u l=180n
M398 nw43 t153 vdd vdd pch w=2u l=180n
CT157 t157 0 0.1f
M399 nw43 t152 t157 0 nch w=1u l=180n
M400 t157 t153 0 0 nch w=1u l=180n
Cnw43 nw43 0 2f
M401 nw44 na6 vdd vdd pch w=2u l=180n
M402 nw44 nb6 vdd vdd pch w=2u l=180n
CT158 t158 0 0.1f
M403 nw44 na6 t158 0 nch w=1u l=180n
M404 t158 nb6 0 0 nch w=1u l=180n
Cnw44 nw44 0 2f
M405 nw45 nw42 vdd vdd pch w=2u l=180n
M406 nw45 nw39 vdd vdd pch w=2u l=180n
CT159 t159 0 0.1f
M407 nw45 nw42 t159 0 nch w=1u l=180n
M408 t159 nw39 0 0 nch w=1u l=180n
Cnw45 nw45 0 2f
M409 nw46 nw44 vdd vdd pch w=2u l=180n
M410 nw46 nw45 vdd vdd pch w=2u l=180n
CT160 t160 0 0.1f
M411 nw46 nw44 t160 0 nch w=1u l=180n
M412 t160 nw45 0 0 nch w=1u l=180n
Cnw46 nw46 0 2f
CT161 t161 0 0.1f
M413 t161 nw43 vdd vdd pch w=2u l=180n
M414 t161 nw43 0 0 nch w=1u l=180n
M415 ns6 t161 vdd vdd pch w=2u l=180n
M416 ns6 t161 0 0 nch w=1u l=180n
Cns6 ns6 0 2f
CT162 t162 0 0.1f
CT163 t163 0 0.1f
CT164 t164 0 0.1f
M417 t162 nw41 vdd vdd pch w=2u l=180n
M418 t162 nw43 vdd vdd pch w=2u l=180n
CT165 t165 0 0.1f
M419 t162 nw41 t165 0 nch w=1u l=180n
M420 t165 nw43 0 0 nch w=1u l=180n
M421 t163 nw41 vdd vdd pch w=2u l=180n
M422 t163 t162 vdd vdd pch w=2u l=180n
CT166 t166 0 0.1f
M423 t163 nw41 t166 0 nch w=1u l=180n
M424 t166 t162 0 0 nch w=1u l=180n
M425 t164 nw43 vdd vdd pch w=2u l=180n
M426 t164 t162 vdd vdd pch w=2u l=180n
CT167 t167 0 0.1f
M427 t164 nw43 t167 0 nch w=1u l=180n
M428 t167 t162 0 0 nch w=1u l=180n
M429 nw48 t163 vdd vdd pch w=2u l=180n
M430 nw48 t164 vdd vdd pch w=2u l=180n
CT168 t168 0 0.1f
M431 nw48 t163 t168 0 nch w=1u l=180n
M432 t168 t164 0 0 nch w=1u l=180n
Cnw48 nw48 0 2f
CT169 t169 0 0.1f
CT170 t170 0 0.1f
CT171 t171 0 0.1f
M433 t169 na7 vdd vdd pch w=2u l=180n
M434 t169 nb7 vdd vdd pch w=2u l=180n
CT172 t172 0 0.1f
M435 t169 na7 t172 0 nch w=1u l=180n
M436 t172 nb7 0 0 nch w=1u l=180n
M437 t170 na7 vdd vdd pch w=2u l=180n
M438 t170 t169 vdd vdd pch w=2u l=180n
CT173 t173 0 0.1f
M439 t170 na7 t173 0 nch w=1u l=180n
M440 t173 t169 0 0 nch w=1u l=180n
M441 t171 nb7 vdd vdd pch w=2u l=180n
M442 t171 t169 vdd vdd pch w=2u l=180n
CT174 t174 0 0.1f
M443 t171 nb7 t174 0 nch w=1u l=180n
M444 t174 t169 0 0 nch w=1u l=180n
M445 nw49 t170 vdd vdd pch w=2u l=180n
M446 nw49 t171 vdd vdd pch w=2u l=180n
CT175 t175 0 0.1f
M447 nw49 t170 t175 0 nch w=1u l=180n
M448 t175 t171 0 0 nch w=1u l=180n
Cnw49 nw49 0 2f
CT176 t176 0 0.1f
CT177 t177 0 0.1f
CT178 t178 0 0.1f
M449 t176 nw49 vdd vdd pch w=2u l=180n
M450 t176 nw46 vdd vdd pch w=2u l=180n
CT179 t179 0 0.1f
M451 t176 nw49 t179 0 nch w=1u l=180n
M452 t179 nw46 0 0 nch w=1u l=180n
M453 t177 nw49 vdd vdd pch w=2u l=180n
M454 t177 t176 vdd vdd pch w=2u l=180n
CT180 t180 0 0.1f
M455 t177 nw49 t180 0 nch w=1u l=180n
M456 t180 t176 0 0 nch w=1u l=180n
M457 t178 nw46 vdd vdd pch w=2u l=180n
M458 t178 t176 vdd vdd pch w=2u l=180n
CT181 t181 0 0.1f
M459 t178 nw46 t181 0 nch w=1u l=180n
M460 t181 t176 0 0 nch w=1u l=180n
M461 nw50 t177 vdd vdd pch w=2u l=180n
M462 nw50 t178 vdd vdd pch w=2u l=180n
CT182 t182 0 0.1f
M463 nw50 t177 t182 0 nch w=1u l=180n
M464 t182 t178 0 0 nch w=1u l=180n
Cnw50 nw50 0 2f
M465 nw51 na7 vdd vdd pch w=2u l=180n
M466 nw51 nb7 vdd vdd pch w=2u l=180n
CT183 t183 0 0.1f
M467 nw51 na7 t183 0 nch w=1u l=180n
M468 t183 nb7 0 0 nch w=1u l=180n
Cnw51 nw51 0 2f
M469 nw52 nw49 vdd vdd pch w=2u l=180n
M470 nw52 nw46 vdd vdd pch w=2u l=180n
CT184 t184 0 0.1f
M471 nw52 nw49 t184 0 nch w=1u l=180n
M472 t184 nw46 0 0 nch w=1u l=180n
Cnw52 nw52 0 2f
M473 nw53 nw51 vdd vdd pch w=2u l=180n
M474 nw53 nw52 vdd vdd pch w=2u l=180n
CT185 t185 0 0.1f
M475 nw53 nw51 t185 0 nch w=1u l=180n
M476 t185 nw52 0 0 nch w=1u l=180n
Cnw53 nw53 0 2f
CT186 t186 0 0.1f
M477 t186 nw50 vdd vdd pch w=2u l=180n
M478 t186 nw50 0 0 nch w=1u l=180n
M479 ns7 t186 vdd vdd pch w=2u l=180n
M480 ns7 t186 0 0 nch w=1u l=180n
Cns7 ns7 0 2f
CT187 t187 0 0.1f
CT188 t188 0 0.1f
CT189 t189 0 0.1f
M481 t187 nw48 vdd vdd pch w=2u l=180n
M482 t187 nw50 vdd vdd pch w=2u l=180n
CT190 t190 0 0.1f
M483 t187 nw48 t190 0 nch w=1u l=180n
M484 t190 nw50 0 0 nch w=1u l=180n
M485 t188 nw48 vdd vdd pch w=2u l=180n
M486 t188 t187 vdd vdd pch w=2u l=180n
CT191 t191 0 0.1f
M487 t188 nw48 t191 0 nch w=1u l=180n
M488 t191 t187 0 0 nch w=1u l=180n
M489 t189 nw50 vdd vdd pch w=2u l=180n
M490 t189 t187 vdd vdd pch w=2u l=180n
CT192 t192 0 0.1f
M491 t189 nw50 t192 0 nch w=1u l=180n
M492 t192 t187 0 0 nch w=1u l=180n
M493 nw55 t188 vdd vdd pch w=2u l=180n
M494 nw55 t189 vdd vdd pch w=2u l=180n
CT193 t193 0 0.1f
M495 nw55 t188 t193 0 nch w=1u l=180n
M496 t193 t189 0 0 nch w=1u l=180n
Cnw55 nw55 0 2f
CT194 t194 0 0.1f
CT195 t195 0 0.1f
CT196 t196 0 0.1f
M497 t194 na8 vdd vdd pch w=2u l=180n
M498 t194 nb8 vdd vdd pch w=2u l=180n
CT197 t197 0 0.1f
M499 t194 na8 t197 0 nch w=1u l=180n
M500 t197 nb8 0 0 nch w=1u l=180n
M501 t195 na8 vdd vdd pch w=2u l=180n
M502 t195 t194 vdd vdd pch w=2u l=180n
CT198 t198 0 0.1f
M503 t195 na8 t198 0 nch w=1u l=180n
M504 t198 t194 0 0 nch w=1u l=180n
M505 t196 nb8 vdd vdd pch w=2u l=180n
M506 t196 t194 vdd vdd pch w=2u l=180n
CT199 t199 0 0.1f
M507 t196 nb8 t199 0 nch w=1u l=180n
M508 t199 t194 0 0 nch w=1u l=180n
M509 nw56 t195 vdd vdd pch w=2u l=180n
M510 nw56 t196 vdd vdd pch w=2u l=180n
CT200 t200 0 0.1f
M511 nw56 t195 t200 0 nch w=1u l=180n
M512 t200 t196 0 0 nch w=1u l=180n
Cnw56 nw56 0 2f
CT201 t201 0 0.1f
CT202 t202 0 0.1f
CT203 t203 0 0.1f
M513 t201 nw56 vdd vdd pch w=2u l=180n
M514 t201 nw53 vdd vdd pch w=2u l=180n
CT204 t204 0 0.1f
M515 t201 nw56 t204 0 nch w=1u l=180n
M516 t204 nw53 0 0 nch w=1u l=180n
M517 t202 nw56 vdd vdd pch w=2u l=180n
M518 t202 t201 vdd vdd pch w=2u l=180n
CT205 t205 0 0.1f
M519 t202 nw56 t205 0 nch w=1u l=180n
M520 t205 t201 0 0 nch w=1u l=180n
M521 t203 nw53 vdd vdd pch w=2u l=180n
M522 t203 t201 vdd vdd pch w=2u l=180n
CT206 t206 0 0.1f
M523 t203 nw53 t206 0 nch w=1u l=180n
M524 t206 t201 0 0 nch w=1u l=180n
M525 nw57 t202 vdd vdd pch w=2u l=180n
M526 nw57 t203 vdd vdd pch w=2u l=180n
CT207 t207 0 0.1f
M527 nw57 t202 t207 0 nch w=1u l=180n
M528 t207 t203 0 0 nch w=1u l=180n
Cnw57 nw57 0 2f
M529 nw58 na8 vdd vdd pch w=2u l=180n
M530 nw58 nb8 vdd vdd pch w=2u l=180n
CT208 t208 0 0.1f
M531 nw58 na8 t208 0 nch w=1u l=180n
M532 t208 nb8 0 0 nch w=1u l=180n
Cnw58 nw58 0 2f
M533 nw59 nw56 vdd vdd pch w=2u l=180n
M534 nw59 nw53 vdd vdd pch w=2u l=180n
CT209 t209 0 0.1f
M535 nw59 nw56 t209 0 nch w=1u l=180n
M536 t209 nw53 0 0 nch w=1u l=180n
Cnw59 nw59 0 2f
M537 nw60 nw58 vdd vdd pch w=2u l=180n
M538 nw60 nw59 vdd vdd pch w=2u l=180n
CT210 t210 0 0.1f
M539 nw60 nw58 t210 0 nch w=1u l=180n
M540 t210 nw59 0 0 nch w=1u l=180n
Cnw60 nw60 0 2f
CT211 t211 0 0.1f
M541 t211 nw57 vdd vdd pch w=2u l=180n
M542 t211 nw57 0 0 nch w=1u l=180n
M543 ns8 t211 vdd vdd pch w=2u l=180n
M544 ns8 t211 0 0 nch w=1u l=180n
Cns8 ns8 0 2f
CT212 t212 0 0.1f
CT213 t213 0 0.1f
CT214 t214 0 0.1f
M545 t212 nw55 vdd vdd pch w=2u l=180n
M546 t212 nw57 vdd vdd pch w=2u l=180n
CT215 t215 0 0.1f
M547 t212 nw55 t215 0 nch w=1u l=180n
M548 t215 nw57 0 0 nch w=1u l=180n
M549 t213 nw55 vdd vdd pch w=2u l=180n
M550 t213 t212 vdd vdd pch w=2u l=180n
CT216 t216 0 0.1f
M551 t213 nw55 t216 0 nch w=1u l=180n
M552 t216 t212 0 0 nch w=1u l=180n
M553 t214 nw57 vdd vdd pch w=2u l=180n
M554 t214 t212 vdd vdd pch w=2u l=180n
CT217 t217 0 0.1f
M555 t214 nw57 t217 0 nch w=1u l=180n
M556 t217 t212 0 0 nch w=1u l=180n
M557 nw62 t213 vdd vdd pch w=2u l=180n
M558 nw62 t214 vdd vdd pch w=2u l=180n
CT218 t218 0 0.1f
M559 nw62 t213 t218 0 nch w=1u l=180n
M560 t218 t214 0 0 nch w=1u l=180n
Cnw62 nw62 0 2f
CT219 t219 0 0.1f
CT220 t220 0 0.1f
CT221 t221 0 0.1f
M561 t219 na9 vdd vdd pch w=2u l=180n
M562 t219 nb9 vdd vdd pch w=2u l=180n
CT222 t222 0 0.1f
M563 t219 na9 t222 0 nch w=1u l=180n
M564 t222 nb9 0 0 nch w=1u l=180n
M565 t220 na9 vdd vdd pch w=2u l=180n
M566 t220 t219 vdd vdd pch w=2u l=180n
CT223 t223 0 0.1f
M567 t220 na9 t223 0 nch w=1u l=180n
M568 t223 t219 0 0 nch w=1u l=180n
M569 t221 nb9 vdd vdd pch w=2u l=180n
M570 t221 t219 vdd vdd pch w=2u l=180n
CT224 t224 0 0.1f
M571 t221 nb9 t224 0 nch w=1u l=180n
M572 t224 t219 0 0 nch w=1u l=180n
M573 nw63 t220 vdd vdd pch w=2u l=180n
M574 nw63 t221 vdd vdd pch w=2u l=180n
CT225 t225 0 0.1f
M575 nw63 t220 t225 0 nch w=1u l=180n
M576 t225 t221 0 0 nch w=1u l=180n
Cnw63 nw63 0 2f
CT226 t226 0 0.1f
CT227 t227 0 0.1f
CT228 t228 0 0.1f
M577 t226 nw63 vdd vdd pch w=2u l=180n
M578 t226 nw60 vdd vdd pch w=2u l=180n
CT229 t229 0 0.1f
M579 t226 nw63 t229 0 nch w=1u l=180n
M580 t229 nw60 0 0 nch w=1u l=180n
M581 t227 nw63 vdd vdd pch w=2u l=180n
M582 t227 t226 vdd vdd pch w=2u l=180n
CT230 t230 0 0.1f
M583 t227 nw63 t230 0 nch w=1u l=180n
M584 t230 t226 0 0 nch w=1u l=180n
M585 t228 nw60 vdd vdd pch w=2u l=180n
M586 t228 t226 vdd vdd pch w=2u l=180n
CT231 t231 0 0.1f
M587 t228 nw60 t231 0 nch w=1u l=180n
M588 t231 t226 0 0 nch w=1u l=180n
M589 nw64 t227 vdd vdd pch w=2u l=180n
M590 nw64 t228 vdd vdd pch w=2u l=180n
CT232 t232 0 0.1f
M591 nw64 t227 t232 0 nch w=1u l=180n
M592 t232 t228 0 0 nch w=1u l=180n
Cnw64 nw64 0 2f
M593 nw65 na9 vdd vdd pch w=2u l=180n
M594 nw65 nb9 vdd vdd pch w=2u l=180n
CT233 t233 0 0.1f
M595 nw65 na9 t233 0 nch w=1u l=180n
M596 t233 nb9 0 0 nch w=1u l=180n
Cnw65 nw65 0 2f
M597 nw66 nw63 vdd vdd pch w=2u l=180n
M598 nw66 nw60 vdd vdd pch w=2u l=180n
CT234 t234 0 0.1f
M599 nw66 nw63 t234 0 nch w=1u l=180n
M600 t234 nw60 0 0 nch w=1u l=180n
Cnw66 nw66 0 2f
M601 nw67 nw65 vdd vdd pch w=2u l=180n
M602 nw67 nw66 vdd vdd pch w=2u l=180n
CT235 t235 0 0.1f
M603 nw67 nw65 t235 0 nch w=1u l=180n
M604 t235 nw66 0 0 nch w=1u l=180n
Cnw67 nw67 0 2f
CT236 t236 0 0.1f
M605 t236 nw64 vdd vdd pch w=2u l=180n
M606 t236 nw64 0 0 nch w=1u l=180n
M607 ns9 t236 vdd vdd pch w=2u l=180n
M608 ns9 t236 0 0 nch w=1u l=180n
Cns9 ns9 0 2f
CT237 t237 0 0.1f
CT238 t238 0 0.1f
CT239 t239 0 0.1f
M609 t237 nw62 vdd vdd pch w=2u l=180n
M610 t237 nw64 vdd vdd pch w=2u l=180n
CT240 t240 0 0.1f
M611 t237 nw62 t240 0 nch w=1u l=180n
M612 t240 nw64 0 0 nch w=1u l=180n
M613 t238 nw62 vdd vdd pch w=2u l=180n
M614 t238 t237 vdd vdd pch w=2u l=180n
CT241 t241 0 0.1f
M615 t238 nw62 t241 0 nch w=1u l=180n
M616 t241 t237 0 0 nch w=1u l=180n
M617 t239 nw64 vdd vdd pch w=2u l=180n
M618 t239 t237 vdd vdd pch w=2u l=180n
CT242 t242 0 0.1f
M619 t239 nw64 t242 0 nch w=1u l=180n
M620 t242 t237 0 0 nch w=1u l=180n
M621 nw69 t238 vdd vdd pch w=2u l=180n
M622 nw69 t239 vdd vdd pch w=2u l=180n
CT243 t243 0 0.1f
M623 nw69 t238 t243 0 nch w=1u l=180n
M624 t243 t239 0 0 nch w=1u l=180n
Cnw69 nw69 0 2f
CT244 t244 0 0.1f
CT245 t245 0 0.1f
CT246 t246 0 0.1f
M625 t244 na10 vdd vdd pch w=2u l=180n
M626 t244 nb10 vdd vdd pch w=2u l=180n
CT247 t247 0 0.1f
M627 t244 na10 t247 0 nch w=1u l=180n
M628 t247 nb10 0 0 nch w=1u l=180n
M629 t245 na10 vdd vdd pch w=2u l=180n
M630 t245 t244 vdd vdd pch w=2u l=180n
CT248 t248 0 0.1f
M631 t245 na10 t248 0 nch w=1u l=180n
M632 t248 t244 0 0 nch w=1u l=180n
M633 t246 nb10 vdd vdd pch w=2u l=180n
M634 t246 t244 vdd vdd pch w=2u l=180n
CT249 t249 0 0.1f
M635 t246 nb10 t249 0 nch w=1u l=180n
M636 t249 t244 0 0 nch w=1u l=180n
M637 nw70 t245 vdd vdd pch w=2u l=180n
M638 nw70 t246 vdd vdd pch w=2u l=180n
CT250 t250 0 0.1f
M639 nw70 t245 t250 0 nch w=1u l=180n
M640 t250 t246 0 0 nch w=1u l=180n
Cnw70 nw70 0 2f
CT251 t251 0 0.1f
CT252 t252 0 0.1f
CT253 t253 0 0.1f
M641 t251 nw70 vdd vdd pch w=2u l=180n
M642 t251 nw67 vdd vdd pch w=2u l=180n
CT254 t254 0 0.1f
M643 t251 nw70 t254 0 nch w=1u l=180n
M644 t254 nw67 0 0 nch w=1u l=180n
M645 t252 nw70 vdd vdd pch w=2u l=180n
M646 t252 t251 vdd vdd pch w=2u l=180n
CT255 t255 0 0.1f
M647 t252 nw70 t255 0 nch w=1u l=180n
M648 t255 t251 0 0 nch w=1u l=180n
M649 t253 nw67 vdd vdd pch w=2u l=180n
M650 t253 t251 vdd vdd pch w=2u l=180n
CT256 t256 0 0.1f
M651 t253 nw67 t256 0 nch w=1u l=180n
M652 t256 t251 0 0 nch w=1u l=180n
M653 nw71 t252 vdd vdd pch w=2u l=180n
M654 nw71 t253 vdd vdd pch w=2u l=180n
CT257 t257 0 0.1f
M655 nw71 t252 t257 0 nch w=1u l=180n
M656 t257 t253 0 0 nch w=1u l=180n
Cnw71 nw71 0 2f
M657 nw72 na10 vdd vdd pch w=2u l=180n
M658 nw72 nb10 vdd vdd pch w=2u l=180n
CT258 t258 0 0.1f
M659 nw72 na10 t258 0 nch w=1u l=180n
M660 t258 nb10 0 0 nch w=1u l=180n
Cnw72 nw72 0 2f
M661 nw73 nw70 vdd vdd pch w=2u l=180n
M662 nw73 nw67 vdd vdd pch w=2u l=180n
CT259 t259 0 0.1f
M663 nw73 nw70 t259 0 nch w=1u l=180n
M664 t259 nw67 0 0 nch w=1u l=180n
Cnw73 nw73 0 2f
M665 nw74 nw72 vdd vdd pch w=2u l=180n
M666 nw74 nw73 vdd vdd pch w=2u l=180n
CT260 t260 0 0.1f
M667 nw74 nw72 t260 0 nch w=1u l=180n
M668 t260 nw73 0 0 nch w=1u l=180n
Cnw74 nw74 0 2f
CT261 t261 0 0.1f
M669 t261 nw71 vdd vdd pch w=2u l=180n
M670 t261 nw71 0 0 nch w=1u l=180n
M671 ns10 t261 vdd vdd pch w=2u l=180n
M672 ns10 t261 0 0 nch w=1u l=180n
Cns10 ns10 0 2f
CT262 t262 0 0.1f
CT263 t263 0 0.1f
CT264 t264 0 0.1f
M673 t262 nw69 vdd vdd pch w=2u l=180n
M674 t262 nw71 vdd vdd pch w=2u l=180n
CT265 t265 0 0.1f
M675 t262 nw69 t265 0 nch w=1u l=180n
M676 t265 nw71 0 0 nch w=1u l=180n
M677 t263 nw69 vdd vdd pch w=2u l=180n
M678 t263 t262 vdd vdd pch w=2u l=180n
CT266 t266 0 0.1f
M679 t263 nw69 t266 0 nch w=1u l=180n
M680 t266 t262 0 0 nch w=1u l=180n
M681 t264 nw71 vdd vdd pch w=2u l=180n
M682 t264 t262 vdd vdd pch w=2u l=180n
CT267 t267 0 0.1f
M683 t264 nw71 t267 0 nch w=1u l=180n
M684 t267 t262 0 0 nch w=1u l=180n
M685 nw76 t263 vdd vdd pch w=2u l=180n
M686 nw76 t264 vdd vdd pch w=2u l=180n
CT268 t268 0 0.1f
M687 nw76 t263 t268 0 nch w=1u l=180n
M688 t268 t264 0 0 nch w=1u l=180n
Cnw76 nw76 0 2f
CT269 t269 0 0.1f
CT270 t270 0 0.1f
CT271 t271 0 0.1f
M689 t269 na11 vdd vdd pch w=2u l=180n
M690 t269 nb11 vdd vdd pch w=2u l=180n
CT272 t272 0 0.1f
M691 t269 na11 t272 0 nch w=1u l=180n
M692 t272 nb11 0 0 nch w=1u l=180n
M693 t270 na11 vdd vdd pch w=2u l=180n
M694 t270 t269 vdd vdd pch w=2u l=180n
CT273 t273 0 0.1f
M695 t270 na11 t273 0 nch w=1u l=180n
M696 t273 t269 0 0 nch w=1u l=180n
M697 t271 nb11 vdd vdd pch w=2u l=180n
M698 t271 t269 vdd vdd pch w=2u l=180n
CT274 t274 0 0.1f
M699 t271 nb11 t274 0 nch w=1u l=180n
M700 t274 t269 0 0 nch w=1u l=180n
M701 nw77 t270 vdd vdd pch w=2u l=180n
M702 nw77 t271 vdd vdd pch w=2u l=180n
CT275 t275 0 0.1f
M703 nw77 t270 t275 0 nch w=1u l=180n
M704 t275 t271 0 0 nch w=1u l=180n
Cnw77 nw77 0 2f
CT276 t276 0 0.1f
CT277 t277 0 0.1f
CT278 t278 0 0.1f
M705 t276 nw77 vdd vdd pch w=2u l=180n
M706 t276 nw74 vdd vdd pch w=2u l=180n
CT279 t279 0 0.1f
M707 t276 nw77 t279 0 nch w=1u l=180n
M708 t279 nw74 0 0 nch w=1u l=180n
M709 t277 nw77 vdd vdd pch w=2u l=180n
M710 t277 t276 vdd vdd pch w=2u l=180n
CT280 t280 0 0.1f
M711 t277 nw77 t280 0 nch w=1u l=180n
M712 t280 t276 0 0 nch w=1u l=180n
M713 t278 nw74 vdd vdd pch w=2u l=180n
M714 t278 t276 vdd vdd pch w=2u l=180n
CT281 t281 0 0.1f
M715 t278 nw74 t281 0 nch w=1u l=180n
M716 t281 t276 0 0 nch w=1u l=180n
M717 nw78 t277 vdd vdd pch w=2u l=180n
M718 nw78 t278 vdd vdd pch w=2u l=180n
CT282 t282 0 0.1f
M719 nw78 t277 t282 0 nch w=1u l=180n
M720 t282 t278 0 0 nch w=1u l=180n
Cnw78 nw78 0 2f
M721 nw79 na11 vdd vdd pch w=2u l=180n
M722 nw79 nb11 vdd vdd pch w=2u l=180n
CT283 t283 0 0.1f
M723 nw79 na11 t283 0 nch w=1u l=180n
M724 t283 nb11 0 0 nch w=1u l=180n
Cnw79 nw79 0 2f
M725 nw80 nw77 vdd vdd pch w=2u l=180n
M726 nw80 nw74 vdd vdd pch w=2u l=180n
CT284 t284 0 0.1f
M727 nw80 nw77 t284 0 nch w=1u l=180n
M728 t284 nw74 0 0 nch w=1u l=180n
Cnw80 nw80 0 2f
M729 nw81 nw79 vdd vdd pch w=2u l=180n
M730 nw81 nw80 vdd vdd pch w=2u l=180n
CT285 t285 0 0.1f
M731 nw81 nw79 t285 0 nch w=1u l=180n
M732 t285 nw80 0 0 nch w=1u l=180n
Cnw81 nw81 0 2f
CT286 t286 0 0.1f
M733 t286 nw78 vdd vdd pch w=2u l=180n
M734 t286 nw78 0 0 nch w=1u l=180n
M735 ns11 t286 vdd vdd pch w=2u l=180n
M736 ns11 t286 0 0 nch w=1u l=180n
Cns11 ns11 0 2f
CT287 t287 0 0.1f
CT288 t288 0 0.1f
CT289 t289 0 0.1f
M737 t287 nw76 vdd vdd pch w=2u l=180n
M738 t287 nw78 vdd vdd pch w=2u l=180n
CT290 t290 0 0.1f
M739 t287 nw76 t290 0 nch w=1u l=180n
M740 t290 nw78 0 0 nch w=1u l=180n
M741 t288 nw76 vdd vdd pch w=2u l=180n
M742 t288 t287 vdd vdd pch w=2u l=180n
CT291 t291 0 0.1f
M743 t288 nw76 t291 0 nch w=1u l=180n
M744 t291 t287 0 0 nch w=1u l=180n
M745 t289 nw78 vdd vdd pch w=2u l=180n
M746 t289 t287 vdd vdd pch w=2u l=180n
CT292 t292 0 0.1f
M747 t289 nw78 t292 0 nch w=1u l=180n
M748 t292 t287 0 0 nch w=1u l=180n
M749 nw83 t288 vdd vdd pch w=2u l=180n
M750 nw83 t289 vdd vdd pch w=2u l=180n
CT293 t293 0 0.1f
M751 nw83 t288 t293 0 nch w=1u l=180n
M752 t293 t289 0 0 nch w=1u l=180n
Cnw83 nw83 0 2f
CT294 t294 0 0.1f
CT295 t295 0 0.1f
CT296 t296 0 0.1f
M753 t294 na11 vdd vdd pch w=2u l=180n
M754 t294 nb11 vdd vdd pch w=2u l=180n
CT297 t297 0 0.1f
M755 t294 na11 t297 0 nch w=1u l=180n
M756 t297 nb11 0 0 nch w=1u l=180n
M757 t295 na11 vdd vdd pch w=2u l=180n
M758 t295 t294 vdd vdd pch w=2u l=180n
CT298 t298 0 0.1f
M759 t295 na11 t298 0 nch w=1u l=180n
M760 t298 t294 0 0 nch w=1u l=180n
M761 t296 nb11 vdd vdd pch w=2u l=180n
M762 t296 t294 vdd vdd pch w=2u l=180n
CT299 t299 0 0.1f
M763 t296 nb11 t299 0 nch w=1u l=180n
M764 t299 t294 0 0 nch w=1u l=180n
CT300 t300 0 0.1f
M765 t300 t295 vdd vdd pch w=2u l=180n
M766 t300 t296 vdd vdd pch w=2u l=180n
CT301 t301 0 0.1f
M767 t300 t295 t301 0 nch w=1u l=180n
M768 t301 t296 0 0 nch w=1u l=180n
M769 nw84 t300 vdd vdd pch w=2u l=180n
M770 nw84 t300 0 0 nch w=1u l=180n
Cnw84 nw84 0 2f
M771 nw85 nb11 vdd vdd pch w=2u l=180n
M772 nw85 nb11 0 0 nch w=1u l=180n
Cnw85 nw85 0 2f
CT302 t302 0 0.1f
M773 t302 na11 vdd vdd pch w=2u l=180n
M774 t302 nw85 vdd vdd pch w=2u l=180n
CT303 t303 0 0.1f
M775 t302 na11 t303 0 nch w=1u l=180n
M776 t303 nw85 0 0 nch w=1u l=180n
M777 nw86 t302 vdd vdd pch w=2u l=180n
M778 nw86 t302 0 0 nch w=1u l=180n
Cnw86 nw86 0 2f
CT304 t304 0 0.1f
CT305 t305 0 0.1f
CT306 t306 0 0.1f
M779 t304 na10 vdd vdd pch w=2u l=180n
M780 t304 nb10 vdd vdd pch w=2u l=180n
CT307 t307 0 0.1f
M781 t304 na10 t307 0 nch w=1u l=180n
M782 t307 nb10 0 0 nch w=1u l=180n
M783 t305 na10 vdd vdd pch w=2u l=180n
M784 t305 t304 vdd vdd pch w=2u l=180n
CT308 t308 0 0.1f
M785 t305 na10 t308 0 nch w=1u l=180n
M786 t308 t304 0 0 nch w=1u l=180n
M787 t306 nb10 vdd vdd pch w=2u l=180n
M788 t306 t304 vdd vdd pch w=2u l=180n
CT309 t309 0 0.1f
M789 t306 nb10 t309 0 nch w=1u l=180n
M790 t309 t304 0 0 nch w=1u l=180n
CT310 t310 0 0.1f
M791 t310 t305 vdd vdd pch w=2u l=180n
M792 t310 t306 vdd vdd pch w=2u l=180n
CT311 t311 0 0.1f
M793 t310 t305 t311 0 nch w=1u l=180n
M794 t311 t306 0 0 nch w=1u l=180n
M795 nw87 t310 vdd vdd pch w=2u l=180n
M796 nw87 t310 0 0 nch w=1u l=180n
Cnw87 nw87 0 2f
M797 nw88 nb10 vdd vdd pch w=2u l=180n
M798 nw88 nb10 0 0 nch w=1u l=180n
Cnw88 nw88 0 2f
CT312 t312 0 0.1f
M799 t312 na10 vdd vdd pch w=2u l=180n
M800 t312 nw88 vdd vdd pch w=2u l=180n
CT313 t313 0 0.1f
M801 t312 na10 t313 0 nch w=1u l=180n
M802 t313 nw88 0 0 nch w=1u l=180n
M803 nw89 t312 vdd vdd pch w=2u l=180n
M804 nw89 t312 0 0 nch w=1u l=180n
Cnw89 nw89 0 2f
CT314 t314 0 0.1f
M805 t314 nw84 vdd vdd pch w=2u l=180n
M806 t314 nw89 vdd vdd pch w=2u l=180n
CT315 t315 0 0.1f
M807 t314 nw84 t315 0 nch w=1u l=180n
M808 t315 nw89 0 0 nch w=1u l=180n
M809 nw90 t314 vdd vdd pch w=2u l=180n
M810 nw90 t314 0 0 nch w=1u l=180n
Cnw90 nw90 0 2f
CT316 t316 0 0.1f
M811 t316 nw86 0 0 nch w=1u l=180n
M812 t316 nw90 0 0 nch w=1u l=180n
CT317 t317 0 0.1f
M813 t317 nw86 vdd vdd pch w=2u l=180n
M814 t316 nw90 t317 vdd pch w=2u l=180n
M815 nw91 t316 vdd vdd pch w=2u l=180n
M816 nw91 t316 0 0 nch w=1u l=180n
Cnw91 nw91 0 2f
CT318 t318 0 0.1f
M817 t318 nw84 vdd vdd pch w=2u l=180n
M818 t318 nw87 vdd vdd pch w=2u l=180n
CT319 t319 0 0.1f
M819 t318 nw84 t319 0 nch w=1u l=180n
M820 t319 nw87 0 0 nch w=1u l=180n
M821 nw92 t318 vdd vdd pch w=2u l=180n
M822 nw92 t318 0 0 nch w=1u l=180n
Cnw92 nw92 0 2f
CT320 t320 0 0.1f
CT321 t321 0 0.1f
CT322 t322 0 0.1f
M823 t320 na9 vdd vdd pch w=2u l=180n
M824 t320 nb9 vdd vdd pch w=2u l=180n
CT323 t323 0 0.1f
M825 t320 na9 t323 0 nch w=1u l=180n
M826 t323 nb9 0 0 nch w=1u l=180n
M827 t321 na9 vdd vdd pch w=2u l=180n
M828 t321 t320 vdd vdd pch w=2u l=180n
CT324 t324 0 0.1f
M829 t321 na9 t324 0 nch w=1u l=180n
M830 t324 t320 0 0 nch w=1u l=180n
M831 t322 nb9 vdd vdd pch w=2u l=180n
M832 t322 t320 vdd vdd pch w=2u l=180n
CT325 t325 0 0.1f
M833 t322 nb9 t325 0 nch w=1u l=180n
M834 t325 t320 0 0 nch w=1u l=180n
CT326 t326 0 0.1f
M835 t326 t321 vdd vdd pch w=2u l=180n
M836 t326 t322 vdd vdd pch w=2u l=180n
CT327 t327 0 0.1f
M837 t326 t321 t327 0 nch w=1u l=180n
M838 t327 t322 0 0 nch w=1u l=180n
M839 nw93 t326 vdd vdd pch w=2u l=180n
M840 nw93 t326 0 0 nch w=1u l=180n
Cnw93 nw93 0 2f
M841 nw94 nb9 vdd vdd pch w=2u l=180n
M842 nw94 nb9 0 0 nch w=1u l=180n
Cnw94 nw94 0 2f
CT328 t328 0 0.1f
M843 t328 na9 vdd vdd pch w=2u l=180n
M844 t328 nw94 vdd vdd pch w=2u l=180n
CT329 t329 0 0.1f
M845 t328 na9 t329 0 nch w=1u l=180n
M846 t329 nw94 0 0 nch w=1u l=180n
M847 nw95 t328 vdd vdd pch w=2u l=180n
M848 nw95 t328 0 0 nch w=1u l=180n
Cnw95 nw95 0 2f
CT330 t330 0 0.1f
M849 t330 nw92 vdd vdd pch w=2u l=180n
M850 t330 nw95 vdd vdd pch w=2u l=180n
CT331 t331 0 0.1f
M851 t330 nw92 t331 0 nch w=1u l=180n
M852 t331 nw95 0 0 nch w=1u l=180n
M853 nw96 t330 vdd vdd pch w=2u l=180n
M854 nw96 t330 0 0 nch w=1u l=180n
Cnw96 nw96 0 2f
CT332 t332 0 0.1f
M855 t332 nw91 0 0 nch w=1u l=180n
M856 t332 nw96 0 0 nch w=1u l=180n
CT333 t333 0 0.1f
M857 t333 nw91 vdd vdd pch w=2u l=180n
M858 t332 nw96 t333 vdd pch w=2u l=180n
M859 nw97 t332 vdd vdd pch w=2u l=180n
M860 nw97 t332 0 0 nch w=1u l=180n
Cnw97 nw97 0 2f
CT334 t334 0 0.1f
M861 t334 nw92 vdd vdd pch w=2u l=180n
M862 t334 nw93 vdd vdd pch w=2u l=180n
CT335 t335 0 0.1f
M863 t334 nw92 t335 0 nch w=1u l=180n
M864 t335 nw93 0 0 nch w=1u l=180n
M865 nw98 t334 vdd vdd pch w=2u l=180n
M866 nw98 t334 0 0 nch w=1u l=180n
Cnw98 nw98 0 2f
CT336 t336 0 0.1f
CT337 t337 0 0.1f
CT338 t338 0 0.1f
M867 t336 na8 vdd vdd pch w=2u l=180n
M868 t336 nb8 vdd vdd pch w=2u l=180n
CT339 t339 0 0.1f
M869 t336 na8 t339 0 nch w=1u l=180n
M870 t339 nb8 0 0 nch w=1u l=180n
M871 t337 na8 vdd vdd pch w=2u l=180n
M872 t337 t336 vdd vdd pch w=2u l=180n
CT340 t340 0 0.1f
M873 t337 na8 t340 0 nch w=1u l=180n
M874 t340 t336 0 0 nch w=1u l=180n
M875 t338 nb8 vdd vdd pch w=2u l=180n
M876 t338 t336 vdd vdd pch w=2u l=180n
CT341 t341 0 0.1f
M877 t338 nb8 t341 0 nch w=1u l=180n
M878 t341 t336 0 0 nch w=1u l=180n
CT342 t342 0 0.1f
M879 t342 t337 vdd vdd pch w=2u l=180n
M880 t342 t338 vdd vdd pch w=2u l=180n
CT343 t343 0 0.1f
M881 t342 t337 t343 0 nch w=1u l=180n
M882 t343 t338 0 0 nch w=1u l=180n
M883 nw99 t342 vdd vdd pch w=2u l=180n
M884 nw99 t342 0 0 nch w=1u l=180n
Cnw99 nw99 0 2f
M885 nw100 nb8 vdd vdd pch w=2u l=180n
M886 nw100 nb8 0 0 nch w=1u l=180n
Cnw100 nw100 0 2f
CT344 t344 0 0.1f
M887 t344 na8 vdd vdd pch w=2u l=180n
M888 t344 nw100 vdd vdd pch w=2u l=180n
CT345 t345 0 0.1f
M889 t344 na8 t345 0 nch w=1u l=180n
M890 t345 nw100 0 0 nch w=1u l=180n
M891 nw101 t344 vdd vdd pch w=2u l=180n
M892 nw101 t344 0 0 nch w=1u l=180n
Cnw101 nw101 0 2f
CT346 t346 0 0.1f
M893 t346 nw98 vdd vdd pch w=2u l=180n
M894 t346 nw101 vdd vdd pch w=2u l=180n
CT347 t347 0 0.1f
M895 t346 nw98 t347 0 nch w=1u l=180n
M896 t347 nw101 0 0 nch w=1u l=180n
M897 nw102 t346 vdd vdd pch w=2u l=180n
M898 nw102 t346 0 0 nch w=1u l=180n
Cnw102 nw102 0 2f
CT348 t348 0 0.1f
M899 t348 nw97 0 0 nch w=1u l=180n
M900 t348 nw102 0 0 nch w=1u l=180n
CT349 t349 0 0.1f
M901 t349 nw97 vdd vdd pch w=2u l=180n
M902 t348 nw102 t349 vdd pch w=2u l=180n
M903 nw103 t348 vdd vdd pch w=2u l=180n
M904 nw103 t348 0 0 nch w=1u l=180n
Cnw103 nw103 0 2f
CT350 t350 0 0.1f
M905 t350 nw98 vdd vdd pch w=2u l=180n
M906 t350 nw99 vdd vdd pch w=2u l=180n
CT351 t351 0 0.1f
M907 t350 nw98 t351 0 nch w=1u l=180n
M908 t351 nw99 0 0 nch w=1u l=180n
M909 nw104 t350 vdd vdd pch w=2u l=180n
M910 nw104 t350 0 0 nch w=1u l=180n
Cnw104 nw104 0 2f
CT352 t352 0 0.1f
CT353 t353 0 0.1f
CT354 t354 0 0.1f
M911 t352 na7 vdd vdd pch w=2u l=180n
M912 t352 nb7 vdd vdd pch w=2u l=180n
CT355 t355 0 0.1f
M913 t352 na7 t355 0 nch w=1u l=180n
M914 t355 nb7 0 0 nch w=1u l=180n
M915 t353 na7 vdd vdd pch w=2u l=180n
M916 t353 t352 vdd vdd pch w=2u l=180n
CT356 t356 0 0.1f
M917 t353 na7 t356 0 nch w=1u l=180n
M918 t356 t352 0 0 nch w=1u l=180n
M919 t354 nb7 vdd vdd pch w=2u l=180n
M920 t354 t352 vdd vdd pch w=2u l=180n
CT357 t357 0 0.1f
M921 t354 nb7 t357 0 nch w=1u l=180n
M922 t357 t352 0 0 nch w=1u l=180n
CT358 t358 0 0.1f
M923 t358 t353 vdd vdd pch w=2u l=180n
M924 t358 t354 vdd vdd pch w=2u l=180n
CT359 t359 0 0.1f
M925 t358 t353 t359 0 nch w=1u l=180n
M926 t359 t354 0 0 nch w=1u l=180n
M927 nw105 t358 vdd vdd pch w=2u l=180n
M928 nw105 t358 0 0 nch w=1u l=180n
Cnw105 nw105 0 2f
M929 nw106 nb7 vdd vdd pch w=2u l=180n
M930 nw106 nb7 0 0 nch w=1u l=180n
Cnw106 nw106 0 2f
CT360 t360 0 0.1f
M931 t360 na7 vdd vdd pch w=2u l=180n
M932 t360 nw106 vdd vdd pch w=2u l=180n
CT361 t361 0 0.1f
M933 t360 na7 t361 0 nch w=1u l=180n
M934 t361 nw106 0 0 nch w=1u l=180n
M935 nw107 t360 vdd vdd pch w=2u l=180n
M936 nw107 t360 0 0 nch w=1u l=180n
Cnw107 nw107 0 2f
CT362 t362 0 0.1f
M937 t362 nw104 vdd vdd pch w=2u l=180n
M938 t362 nw107 vdd vdd pch w=2u l=180n
CT363 t363 0 0.1f
M939 t362 nw104 t363 0 nch w=1u l=180n
M940 t363 nw107 0 0 nch w=1u l=180n
M941 nw108 t362 vdd vdd pch w=2u l=180n
M942 nw108 t362 0 0 nch w=1u l=180n
Cnw108 nw108 0 2f
CT364 t364 0 0.1f
M943 t364 nw103 0 0 nch w=1u l=180n
M944 t364 nw108 0 0 nch w=1u l=180n
CT365 t365 0 0.1f
M945 t365 nw103 vdd vdd pch w=2u l=180n
M946 t364 nw108 t365 vdd pch w=2u l=180n
M947 nw109 t364 vdd vdd pch w=2u l=180n
M948 nw109 t364 0 0 nch w=1u l=180n
Cnw109 nw109 0 2f
CT366 t366 0 0.1f
M949 t366 nw104 vdd vdd pch w=2u l=180n
M950 t366 nw105 vdd vdd pch w=2u l=180n
CT367 t367 0 0.1f
M951 t366 nw104 t367 0 nch w=1u l=180n
M952 t367 nw105 0 0 nch w=1u l=180n
M953 nw110 t366 vdd vdd pch w=2u l=180n
M954 nw110 t366 0 0 nch w=1u l=180n
Cnw110 nw110 0 2f
CT368 t368 0 0.1f
CT369 t369 0 0.1f
CT370 t370 0 0.1f
M955 t368 na6 vdd vdd pch w=2u l=180n
M956 t368 nb6 vdd vdd pch w=2u l=180n
CT371 t371 0 0.1f
M957 t368 na6 t371 0 nch w=1u l=180n
M958 t371 nb6 0 0 nch w=1u l=180n
M959 t369 na6 vdd vdd pch w=2u l=180n
M960 t369 t368 vdd vdd pch w=2u l=180n
CT372 t372 0 0.1f
M961 t369 na6 t372 0 nch w=1u l=180n
M962 t372 t368 0 0 nch w=1u l=180n
M963 t370 nb6 vdd vdd pch w=2u l=180n
M964 t370 t368 vdd vdd pch w=2u l=180n
CT373 t373 0 0.1f
M965 t370 nb6 t373 0 nch w=1u l=180n
M966 t373 t368 0 0 nch w=1u l=180n
CT374 t374 0 0.1f
M967 t374 t369 vdd vdd pch w=2u l=180n
M968 t374 t370 vdd vdd pch w=2u l=180n
CT375 t375 0 0.1f
M969 t374 t369 t375 0 nch w=1u l=180n
M970 t375 t370 0 0 nch w=1u l=180n
M971 nw111 t374 vdd vdd pch w=2u l=180n
M972 nw111 t374 0 0 nch w=1u l=180n
Cnw111 nw111 0 2f
M973 nw112 nb6 vdd vdd pch w=2u l=180n
M974 nw112 nb6 0 0 nch w=1u l=180n
Cnw112 nw112 0 2f
CT376 t376 0 0.1f
M975 t376 na6 vdd vdd pch w=2u l=180n
M976 t376 nw112 vdd vdd pch w=2u l=180n
CT377 t377 0 0.1f
M977 t376 na6 t377 0 nch w=1u l=180n
M978 t377 nw112 0 0 nch w=1u l=180n
M979 nw113 t376 vdd vdd pch w=2u l=180n
M980 nw113 t376 0 0 nch w=1u l=180n
Cnw113 nw113 0 2f
CT378 t378 0 0.1f
M981 t378 nw110 vdd vdd pch w=2u l=180n
M982 t378 nw113 vdd vdd pch w=2u l=180n
CT379 t379 0 0.1f
M983 t378 nw110 t379 0 nch w=1u l=180n
M984 t379 nw113 0 0 nch w=1u l=180n
M985 nw114 t378 vdd vdd pch w=2u l=180n
M986 nw114 t378 0 0 nch w=1u l=180n
Cnw114 nw114 0 2f
CT380 t380 0 0.1f
M987 t380 nw109 0 0 nch w=1u l=180n
M988 t380 nw114 0 0 nch w=1u l=180n
CT381 t381 0 0.1f
M989 t381 nw109 vdd vdd pch w=2u l=180n
M990 t380 nw114 t381 vdd pch w=2u l=180n
M991 nw115 t380 vdd vdd pch w=2u l=180n
M992 nw115 t380 0 0 nch w=1u l=180n
Cnw115 nw115 0 2f
CT382 t382 0 0.1f
M993 t382 nw110 vdd vdd pch w=2u l=180n
M994 t382 nw111 vdd vdd pch w=2u l=180n
CT383 t383 0 0.1f
M995 t382 nw110 t383 0 nch w=1u l=180n
M996 t383 nw111 0 0 nch w=1u l=180n
M997 nw116 t382 vdd vdd pch w=2u l=180n
M998 nw116 t382 0 0 nch w=1u l=180n
Cnw116 nw116 0 2f
CT384 t384 0 0.1f
CT385 t385 0 0.1f
CT386 t386 0 0.1f
M999 t384 na5 vdd vdd pch w=2u l=180n
M1000 t384 nb5 vdd vdd pch w=2u l=180n
CT387 t387 0 0.1f
M1001 t384 na5 t387 0 nch w=1u l=180n
M1002 t387 nb5 0 0 nch w=1u l=180n
M1003 t385 na5 vdd vdd pch w=2u l=180n
M1004 t385 t384 vdd vdd pch w=2u l=180n
CT388 t388 0 0.1f
M1005 t385 na5 t388 0 nch w=1u l=180n
M1006 t388 t384 0 0 nch w=1u l=180n
M1007 t386 nb5 vdd vdd pch w=2u l=180n
M1008 t386 t384 vdd vdd pch w=2u l=180n
CT389 t389 0 0.1f
M1009 t386 nb5 t389 0 nch w=1u l=180n
M1010 t389 t384 0 0 nch w=1u l=180n
CT390 t390 0 0.1f
M1011 t390 t385 vdd vdd pch w=2u l=180n
M1012 t390 t386 vdd vdd pch w=2u l=180n
CT391 t391 0 0.1f
M1013 t390 t385 t391 0 nch w=1u l=180n
M1014 t391 t386 0 0 nch w=1u l=180n
M1015 nw117 t390 vdd vdd pch w=2u l=180n
M1016 nw117 t390 0 0 nch w=1u l=180n
Cnw117 nw117 0 2f
M1017 nw118 nb5 vdd vdd pch w=2u l=180n
M1018 nw118 nb5 0 0 nch w=1u l=180n
Cnw118 nw118 0 2f
CT392 t392 0 0.1f
M1019 t392 na5 vdd vdd pch w=2u l=180n
M1020 t392 nw118 vdd vdd pch w=2u l=180n
CT393 t393 0 0.1f
M1021 t392 na5 t393 0 nch w=1u l=180n
M1022 t393 nw118 0 0 nch w=1u l=180n
M1023 nw119 t392 vdd vdd pch w=2u l=180n
M1024 nw119 t392 0 0 nch w=1u l=180n
Cnw119 nw119 0 2f
CT394 t394 0 0.1f
M1025 t394 nw116 vdd vdd pch w=2u l=180n
M1026 t394 nw119 vdd vdd pch w=2u l=180n
CT395 t395 0 0.1f
M1027 t394 nw116 t395 0 nch w=1u l=180n
M1028 t395 nw119 0 0 nch w=1u l=180n
M1029 nw120 t394 vdd vdd pch w=2u l=180n
M1030 nw120 t394 0 0 nch w=1u l=180n
Cnw120 nw120 0 2f
CT396 t396 0 0.1f
M1031 t396 nw115 0 0 nch w=1u l=180n
M1032 t396 nw120 0 0 nch w=1u l=180n
CT397 t397 0 0.1f
M1033 t397 nw115 vdd vdd pch w=2u l=180n
M1034 t396 nw120 t397 vdd pch w=2u l=180n
M1035 nw121 t396 vdd vdd pch w=2u l=180n
M1036 nw121 t396 0 0 nch w=1u l=180n
Cnw121 nw121 0 2f
CT398 t398 0 0.1f
M1037 t398 nw116 vdd vdd pch w=2u l=180n
M1038 t398 nw117 vdd vdd pch w=2u l=180n
CT399 t399 0 0.1f
M1039 t398 nw116 t399 0 nch w=1u l=180n
M1040 t399 nw117 0 0 nch w=1u l=180n
M1041 nw122 t398 vdd vdd pch w=2u l=180n
M1042 nw122 t398 0 0 nch w=1u l=180n
Cnw122 nw122 0 2f
CT400 t400 0 0.1f
CT401 t401 0 0.1f
CT402 t402 0 0.1f
M1043 t400 na4 vdd vdd pch w=2u l=180n
M1044 t400 nb4 vdd vdd pch w=2u l=180n
CT403 t403 0 0.1f
M1045 t400 na4 t403 0 nch w=1u l=180n
M1046 t403 nb4 0 0 nch w=1u l=180n
M1047 t401 na4 vdd vdd pch w=2u l=180n
M1048 t401 t400 vdd vdd pch w=2u l=180n
CT404 t404 0 0.1f
M1049 t401 na4 t404 0 nch w=1u l=180n
M1050 t404 t400 0 0 nch w=1u l=180n
M1051 t402 nb4 vdd vdd pch w=2u l=180n
M1052 t402 t400 vdd vdd pch w=2u l=180n
CT405 t405 0 0.1f
M1053 t402 nb4 t405 0 nch w=1u l=180n
M1054 t405 t400 0 0 nch w=1u l=180n
CT406 t406 0 0.1f
M1055 t406 t401 vdd vdd pch w=2u l=180n
M1056 t406 t402 vdd vdd pch w=2u l=180n
CT407 t407 0 0.1f
M1057 t406 t401 t407 0 nch w=1u l=180n
M1058 t407 t402 0 0 nch w=1u l=180n
M1059 nw123 t406 vdd vdd pch w=2u l=180n
M1060 nw123 t406 0 0 nch w=1u l=180n
Cnw123 nw123 0 2f
M1061 nw124 nb4 vdd vdd pch w=2u l=180n
M1062 nw124 nb4 0 0 nch w=1u l=180n
Cnw124 nw124 0 2f
CT408 t408 0 0.1f
M1063 t408 na4 vdd vdd pch w=2u l=180n
M1064 t408 nw124 vdd vdd pch w=2u l=180n
CT409 t409 0 0.1f
M1065 t408 na4 t409 0 nch w=1u l=180n
M1066 t409 nw124 0 0 nch w=1u l=180n
M1067 nw125 t408 vdd vdd pch w=2u l=180n
M1068 nw125 t408 0 0 nch w=1u l=180n
Cnw125 nw125 0 2f
CT410 t410 0 0.1f
M1069 t410 nw122 vdd vdd pch w=2u l=180n
M1070 t410 nw125 vdd vdd pch w=2u l=180n
CT411 t411 0 0.1f
M1071 t410 nw122 t411 0 nch w=1u l=180n
M1072 t411 nw125 0 0 nch w=1u l=180n
M1073 nw126 t410 vdd vdd pch w=2u l=180n
M1074 nw126 t410 0 0 nch w=1u l=180n
Cnw126 nw126 0 2f
CT412 t412 0 0.1f
M1075 t412 nw121 0 0 nch w=1u l=180n
M1076 t412 nw126 0 0 nch w=1u l=180n
CT413 t413 0 0.1f
M1077 t413 nw121 vdd vdd pch w=2u l=180n
M1078 t412 nw126 t413 vdd pch w=2u l=180n
M1079 nw127 t412 vdd vdd pch w=2u l=180n
M1080 nw127 t412 0 0 nch w=1u l=180n
Cnw127 nw127 0 2f
CT414 t414 0 0.1f
M1081 t414 nw122 vdd vdd pch w=2u l=180n
M1082 t414 nw123 vdd vdd pch w=2u l=180n
CT415 t415 0 0.1f
M1083 t414 nw122 t415 0 nch w=1u l=180n
M1084 t415 nw123 0 0 nch w=1u l=180n
M1085 nw128 t414 vdd vdd pch w=2u l=180n
M1086 nw128 t414 0 0 nch w=1u l=180n
Cnw128 nw128 0 2f
CT416 t416 0 0.1f
CT417 t417 0 0.1f
CT418 t418 0 0.1f
M1087 t416 na3 vdd vdd pch w=2u l=180n
M1088 t416 nb3 vdd vdd pch w=2u l=180n
CT419 t419 0 0.1f
M1089 t416 na3 t419 0 nch w=1u l=180n
M1090 t419 nb3 0 0 nch w=1u l=180n
M1091 t417 na3 vdd vdd pch w=2u l=180n
M1092 t417 t416 vdd vdd pch w=2u l=180n
CT420 t420 0 0.1f
M1093 t417 na3 t420 0 nch w=1u l=180n
M1094 t420 t416 0 0 nch w=1u l=180n
M1095 t418 nb3 vdd vdd pch w=2u l=180n
M1096 t418 t416 vdd vdd pch w=2u l=180n
CT421 t421 0 0.1f
M1097 t418 nb3 t421 0 nch w=1u l=180n
M1098 t421 t416 0 0 nch w=1u l=180n
CT422 t422 0 0.1f
M1099 t422 t417 vdd vdd pch w=2u l=180n
M1100 t422 t418 vdd vdd pch w=2u l=180n
CT423 t423 0 0.1f
M1101 t422 t417 t423 0 nch w=1u l=180n
M1102 t423 t418 0 0 nch w=1u l=180n
M1103 nw129 t422 vdd vdd pch w=2u l=180n
M1104 nw129 t422 0 0 nch w=1u l=180n
Cnw129 nw129 0 2f
M1105 nw130 nb3 vdd vdd pch w=2u l=180n
M1106 nw130 nb3 0 0 nch w=1u l=180n
Cnw130 nw130 0 2f
CT424 t424 0 0.1f
M1107 t424 na3 vdd vdd pch w=2u l=180n
M1108 t424 nw130 vdd vdd pch w=2u l=180n
CT425 t425 0 0.1f
M1109 t424 na3 t425 0 nch w=1u l=180n
M1110 t425 nw130 0 0 nch w=1u l=180n
M1111 nw131 t424 vdd vdd pch w=2u l=180n
M1112 nw131 t424 0 0 nch w=1u l=180n
Cnw131 nw131 0 2f
CT426 t426 0 0.1f
M1113 t426 nw128 vdd vdd pch w=2u l=180n
M1114 t426 nw131 vdd vdd pch w=2u l=180n
CT427 t427 0 0.1f
M1115 t426 nw128 t427 0 nch w=1u l=180n
M1116 t427 nw131 0 0 nch w=1u l=180n
M1117 nw132 t426 vdd vdd pch w=2u l=180n
M1118 nw132 t426 0 0 nch w=1u l=180n
Cnw132 nw132 0 2f
CT428 t428 0 0.1f
M1119 t428 nw127 0 0 nch w=1u l=180n
M1120 t428 nw132 0 0 nch w=1u l=180n
CT429 t429 0 0.1f
M1121 t429 nw127 vdd vdd pch w=2u l=180n
M1122 t428 nw132 t429 vdd pch w=2u l=180n
M1123 nw133 t428 vdd vdd pch w=2u l=180n
M1124 nw133 t428 0 0 nch w=1u l=180n
Cnw133 nw133 0 2f
CT430 t430 0 0.1f
M1125 t430 nw128 vdd vdd pch w=2u l=180n
M1126 t430 nw129 vdd vdd pch w=2u l=180n
CT431 t431 0 0.1f
M1127 t430 nw128 t431 0 nch w=1u l=180n
M1128 t431 nw129 0 0 nch w=1u l=180n
M1129 nw134 t430 vdd vdd pch w=2u l=180n
M1130 nw134 t430 0 0 nch w=1u l=180n
Cnw134 nw134 0 2f
CT432 t432 0 0.1f
CT433 t433 0 0.1f
CT434 t434 0 0.1f
M1131 t432 na2 vdd vdd pch w=2u l=180n
M1132 t432 nb2 vdd vdd pch w=2u l=180n
CT435 t435 0 0.1f
M1133 t432 na2 t435 0 nch w=1u l=180n
M1134 t435 nb2 0 0 nch w=1u l=180n
M1135 t433 na2 vdd vdd pch w=2u l=180n
M1136 t433 t432 vdd vdd pch w=2u l=180n
CT436 t436 0 0.1f
M1137 t433 na2 t436 0 nch w=1u l=180n
M1138 t436 t432 0 0 nch w=1u l=180n
M1139 t434 nb2 vdd vdd pch w=2u l=180n
M1140 t434 t432 vdd vdd pch w=2u l=180n
CT437 t437 0 0.1f
M1141 t434 nb2 t437 0 nch w=1u l=180n
M1142 t437 t432 0 0 nch w=1u l=180n
CT438 t438 0 0.1f
M1143 t438 t433 vdd vdd pch w=2u l=180n
M1144 t438 t434 vdd vdd pch w=2u l=180n
CT439 t439 0 0.1f
M1145 t438 t433 t439 0 nch w=1u l=180n
M1146 t439 t434 0 0 nch w=1u l=180n
M1147 nw135 t438 vdd vdd pch w=2u l=180n
M1148 nw135 t438 0 0 nch w=1u l=180n
Cnw135 nw135 0 2f
M1149 nw136 nb2 vdd vdd pch w=2u l=180n
M1150 nw136 nb2 0 0 nch w=1u l=180n
Cnw136 nw136 0 2f
CT440 t440 0 0.1f
M1151 t440 na2 vdd vdd pch w=2u l=180n
M1152 t440 nw136 vdd vdd pch w=2u l=180n
CT441 t441 0 0.1f
M1153 t440 na2 t441 0 nch w=1u l=180n
M1154 t441 nw136 0 0 nch w=1u l=180n
M1155 nw137 t440 vdd vdd pch w=2u l=180n
M1156 nw137 t440 0 0 nch w=1u l=180n
Cnw137 nw137 0 2f
CT442 t442 0 0.1f
M1157 t442 nw134 vdd vdd pch w=2u l=180n
M1158 t442 nw137 vdd vdd pch w=2u l=180n
CT443 t443 0 0.1f
M1159 t442 nw134 t443 0 nch w=1u l=180n
M1160 t443 nw137 0 0 nch w=1u l=180n
M1161 nw138 t442 vdd vdd pch w=2u l=180n
M1162 nw138 t442 0 0 nch w=1u l=180n
Cnw138 nw138 0 2f
CT444 t444 0 0.1f
M1163 t444 nw133 0 0 nch w=1u l=180n
M1164 t444 nw138 0 0 nch w=1u l=180n
CT445 t445 0 0.1f
M1165 t445 nw133 vdd vdd pch w=2u l=180n
M1166 t444 nw138 t445 vdd pch w=2u l=180n
M1167 nw139 t444 vdd vdd pch w=2u l=180n
M1168 nw139 t444 0 0 nch w=1u l=180n
Cnw139 nw139 0 2f
CT446 t446 0 0.1f
M1169 t446 nw134 vdd vdd pch w=2u l=180n
M1170 t446 nw135 vdd vdd pch w=2u l=180n
CT447 t447 0 0.1f
M1171 t446 nw134 t447 0 nch w=1u l=180n
M1172 t447 nw135 0 0 nch w=1u l=180n
M1173 nw140 t446 vdd vdd pch w=2u l=180n
M1174 nw140 t446 0 0 nch w=1u l=180n
Cnw140 nw140 0 2f
CT448 t448 0 0.1f
CT449 t449 0 0.1f
CT450 t450 0 0.1f
M1175 t448 na1 vdd vdd pch w=2u l=180n
M1176 t448 nb1 vdd vdd pch w=2u l=180n
CT451 t451 0 0.1f
M1177 t448 na1 t451 0 nch w=1u l=180n
M1178 t451 nb1 0 0 nch w=1u l=180n
M1179 t449 na1 vdd vdd pch w=2u l=180n
M1180 t449 t448 vdd vdd pch w=2u l=180n
CT452 t452 0 0.1f
M1181 t449 na1 t452 0 nch w=1u l=180n
M1182 t452 t448 0 0 nch w=1u l=180n
M1183 t450 nb1 vdd vdd pch w=2u l=180n
M1184 t450 t448 vdd vdd pch w=2u l=180n
CT453 t453 0 0.1f
M1185 t450 nb1 t453 0 nch w=1u l=180n
M1186 t453 t448 0 0 nch w=1u l=180n
CT454 t454 0 0.1f
M1187 t454 t449 vdd vdd pch w=2u l=180n
M1188 t454 t450 vdd vdd pch w=2u l=180n
CT455 t455 0 0.1f
M1189 t454 t449 t455 0 nch w=1u l=180n
M1190 t455 t450 0 0 nch w=1u l=180n
M1191 nw141 t454 vdd vdd pch w=2u l=180n
M1192 nw141 t454 0 0 nch w=1u l=180n
Cnw141 nw141 0 2f
M1193 nw142 nb1 vdd vdd pch w=2u l=180n
M1194 nw142 nb1 0 0 nch w=1u l=180n
Cnw142 nw142 0 2f
CT456 t456 0 0.1f
M1195 t456 na1 vdd vdd pch w=2u l=180n
M1196 t456 nw142 vdd vdd pch w=2u l=180n
CT457 t457 0 0.1f
M1197 t456 na1 t457 0 nch w=1u l=180n
M1198 t457 nw142 0 0 nch w=1u l=180n
M1199 nw143 t456 vdd vdd pch w=2u l=180n
M1200 nw143 t456 0 0 nch w=1u l=180n
Cnw143 nw143 0 2f
CT458 t458 0 0.1f
M1201 t458 nw140 vdd vdd pch w=2u l=180n
M1202 t458 nw143 vdd vdd pch w=2u l=180n
CT459 t459 0 0.1f
M1203 t458 nw140 t459 0 nch w=1u l=180n
M1204 t459 nw143 0 0 nch w=1u l=180n
M1205 nw144 t458 vdd vdd pch w=2u l=180n
M1206 nw144 t458 0 0 nch w=1u l=180n
Cnw144 nw144 0 2f
CT460 t460 0 0.1f
M1207 t460 nw139 0 0 nch w=1u l=180n
M1208 t460 nw144 0 0 nch w=1u l=180n
CT461 t461 0 0.1f
M1209 t461 nw139 vdd vdd pch w=2u l=180n
M1210 t460 nw144 t461 vdd pch w=2u l=180n
M1211 nw145 t460 vdd vdd pch w=2u l=180n
M1212 nw145 t460 0 0 nch w=1u l=180n
Cnw145 nw145 0 2f
CT462 t462 0 0.1f
M1213 t462 nw140 vdd vdd pch w=2u l=180n
M1214 t462 nw141 vdd vdd pch w=2u l=180n
CT463 t463 0 0.1f
M1215 t462 nw140 t463 0 nch w=1u l=180n
M1216 t463 nw141 0 0 nch w=1u l=180n
M1217 nw146 t462 vdd vdd pch w=2u l=180n
M1218 nw146 t462 0 0 nch w=1u l=180n
Cnw146 nw146 0 2f
CT464 t464 0 0.1f
CT465 t465 0 0.1f
CT466 t466 0 0.1f
M1219 t464 na0 vdd vdd pch w=2u l=180n
M1220 t464 nb0 vdd vdd pch w=2u l=180n
CT467 t467 0 0.1f
M1221 t464 na0 t467 0 nch w=1u l=180n
M1222 t467 nb0 0 0 nch w=1u l=180n
M1223 t465 na0 vdd vdd pch w=2u l=180n
M1224 t465 t464 vdd vdd pch w=2u l=180n
CT468 t468 0 0.1f
M1225 t465 na0 t468 0 nch w=1u l=180n
M1226 t468 t464 0 0 nch w=1u l=180n
M1227 t466 nb0 vdd vdd pch w=2u l=180n
M1228 t466 t464 vdd vdd pch w=2u l=180n
CT469 t469 0 0.1f
M1229 t466 nb0 t469 0 nch w=1u l=180n
M1230 t469 t464 0 0 nch w=1u l=180n
CT470 t470 0 0.1f
M1231 t470 t465 vdd vdd pch w=2u l=180n
M1232 t470 t466 vdd vdd pch w=2u l=180n
CT471 t471 0 0.1f
M1233 t470 t465 t471 0 nch w=1u l=180n
M1234 t471 t466 0 0 nch w=1u l=180n
M1235 nw147 t470 vdd vdd pch w=2u l=180n
M1236 nw147 t470 0 0 nch w=1u l=180n
Cnw147 nw147 0 2f
M1237 nw148 nb0 vdd vdd pch w=2u l=180n
M1238 nw148 nb0 0 0 nch w=1u l=180n
Cnw148 nw148 0 2f
CT472 t472 0 0.1f
M1239 t472 na0 vdd vdd pch w=2u l=180n
M1240 t472 nw148 vdd vdd pch w=2u l=180n
CT473 t473 0 0.1f
M1241 t472 na0 t473 0 nch w=1u l=180n
M1242 t473 nw148 0 0 nch w=1u l=180n
M1243 nw149 t472 vdd vdd pch w=2u l=180n
M1244 nw149 t472 0 0 nch w=1u l=180n
Cnw149 nw149 0 2f
CT474 t474 0 0.1f
M1245 t474 nw146 vdd vdd pch w=2u l=180n
M1246 t474 nw149 vdd vdd pch w=2u l=180n
CT475 t475 0 0.1f
M1247 t474 nw146 t475 0 nch w=1u l=180n
M1248 t475 nw149 0 0 nch w=1u l=180n
M1249 nw150 t474 vdd vdd pch w=2u l=180n
M1250 nw150 t474 0 0 nch w=1u l=180n
Cnw150 nw150 0 2f
CT476 t476 0 0.1f
M1251 t476 nw145 0 0 nch w=1u l=180n
M1252 t476 nw150 0 0 nch w=1u l=180n
CT477 t477 0 0.1f
M1253 t477 nw145 vdd vdd pch w=2u l=180n
M1254 t476 nw150 t477 vdd pch w=2u l=180n
M1255 nw151 t476 vdd vdd pch w=2u l=180n
M1256 nw151 t476 0 0 nch w=1u l=180n
Cnw151 nw151 0 2f
CT478 t478 0 0.1f
M1257 t478 nw146 vdd vdd pch w=2u l=180n
M1258 t478 nw147 vdd vdd pch w=2u l=180n
CT479 t479 0 0.1f
M1259 t478 nw146 t479 0 nch w=1u l=180n
M1260 t479 nw147 0 0 nch w=1u l=180n
M1261 nw152 t478 vdd vdd pch w=2u l=180n
M1262 nw152 t478 0 0 nch w=1u l=180n
Cnw152 nw152 0 2f
CT480 t480 0 0.1f
M1263 t480 nw81 vdd vdd pch w=2u l=180n
M1264 t480 nw81 0 0 nch w=1u l=180n
M1265 ncout t480 vdd vdd pch w=2u l=180n
M1266 ncout t480 0 0 nch w=1u l=180n
Cncout ncout 0 2f
CT481 t481 0 0.1f
M1267 t481 nw83 vdd vdd pch w=2u l=180n
M1268 t481 nw83 0 0 nch w=1u l=180n
M1269 nparity t481 vdd vdd pch w=2u l=180n
M1270 nparity t481 0 0 nch w=1u l=180n
Cnparity nparity 0 2f
CT482 t482 0 0.1f
M1271 t482 nw151 vdd vdd pch w=2u l=180n
M1272 t482 nw151 0 0 nch w=1u l=180n
M1273 na_gt_b t482 vdd vdd pch w=2u l=180n
M1274 na_gt_b t482 0 0 nch w=1u l=180n
Cna_gt_b na_gt_b 0 2f
CT483 t483 0 0.1f
M1275 t483 nw152 vdd vdd pch w=2u l=180n
M1276 t483 nw152 0 0 nch w=1u l=180n
M1277 na_eq_b t483 vdd vdd pch w=2u l=180n
M1278 na_eq_b t483 0 0 nch w=1u l=180n
Cna_eq_b na_eq_b 0 2f
.model nch NMOS (vto=0.45 kp=200u lambda=0.05)
.model pch PMOS (vto=-0.45 kp=100u lambda=0.05)
* outputs: ns0 ns1 ns2 ns3 ns4 ns5 ns6 ns7 ns8 ns9 ns10 ns11 ncout nparity na_gt_b na_eq_b
.end
