* s1488 (s1488: controller, 6 flip-flops, 653 gates): 670 gates, 4844 transistors
VDD vdd 0 DC 1.8
VIN0 ni0 0 PULSE(0 1.8 5e-10 20p 20p 1e-09 2e-09)
VIN1 ni1 0 PULSE(0 1.8 1e-09 20p 20p 2e-09 4e-09)
VIN2 ni2 0 PULSE(0 1.8 2e-09 20p 20p 4e-09 8e-09)
VIN3 nq0 0 PULSE(0 1.8 4e-09 20p 20p 8e-09 1.6e-08)
VIN4 nq1 0 PULSE(0 1.8 8e-09 20p 20p 1.6e-08 3.2e-08)
VIN5 nq2 0 PULSE(0 1.8 1.6e-08 20p 20p 3.2e-08 6.4e-08)
VIN6 nq3 0 PULSE(0 1.8 3.2e-08 20p 20p 6.4e-08 1.28e-07)
VIN7 nq4 0 PULSE(0 1.8 6.4e-08 20p 20p 1.28e-07 2.56e-07)
VIN8 nq5 0 PULSE(0 1.8 1.28e-07 20p 20p 2.56e-07 5.12e-07)
CT1 t1 0 0.1f
CT2 t2 0 0.1f
CT3 t3 0 0.1f
M1 t1 nq0 vdd vdd pch w=2u l=180n
M2 t1 ni0 vdd vdd pch w=2u l=180n
CT4 t4 0 0.1f
M3 t1 nq0 t4 0 nch w=1u l=180n
M4 t4 ni0 0 0 nch w=1u l=180n
M5 t2 nq0 vdd vdd pch w=2u l=180n
M6 t2 t1 vdd vdd pch w=2u l=180n
CT5 t5 0 0.1f
M7 t2 nq0 t5 0 nch w=1u l=180n
M8 t5 t1 0 0 nch w=1u l=180n
M9 t3 ni0 vdd vdd pch w=2u l=180n
M10 t3 t1 vdd vdd pch w=2u l=180n
CT6 t6 0 0.1f
M11 t3 ni0 t6 0 nch w=1u l=180n
M12 t6 t1 0 0 nch w=1u l=180n
M13 nw1 t2 vdd vdd pch w=2u l=180n
M14 nw1 t3 vdd vdd pch w=2u l=180n
CT7 t7 0 0.1f
M15 nw1 t2 t7 0 nch w=1u l=180n
M16 t7 t3 0 0 nch w=1u l=180n
Cnw1 nw1 0 2f
CT8 t8 0 0.1f
M17 t8 ni0 vdd vdd pch w=2u l=180n
M18 t8 nq0 vdd vdd pch w=2u l=180n
CT9 t9 0 0.1f
M19 t8 ni0 t9 0 nch w=1u l=180n
M20 t9 nq0 0 0 nch w=1u l=180n
M21 nw2 t8 vdd vdd pch w=2u l=180n
M22 nw2 t8 0 0 nch w=1u l=180n
Cnw2 nw2 0 2f
CT10 t10 0 0.1f
CT11 t11 0 0.1f
CT12 t12 0 0.1f
M23 t10 nq1 vdd vdd pch w=2u l=180n
M24 t10 nw2 vdd vdd pch w=2u l=180n
CT13 t13 0 0.1f
M25 t10 nq1 t13 0 nch w=1u l=180n
M26 t13 nw2 0 0 nch w=1u l=180n
M27 t11 nq1 vdd vdd pch w=2u l=180n
M28 t11 t10 vdd vdd pch w=2u l=180n
CT14 t14 0 0.1f
M29 t11 nq1 t14 0 nch w=1u l=180n
M30 t14 t10 0 0 nch w=1u l=180n
M31 t12 nw2 vdd vdd pch w=2u l=180n
M32 t12 t10 vdd vdd pch w=2u l=180n
CT15 t15 0 0.1f
M33 t12 nw2 t15 0 nch w=1u l=180n
M34 t15 t10 0 0 nch w=1u l=180n
M35 nw3 t11 vdd vdd pch w=2u l=180n
M36 nw3 t12 vdd vdd pch w=2u l=180n
CT16 t16 0 0.1f
M37 nw3 t11 t16 0 nch w=1u l=180n
M38 t16 t12 0 0 nch w=1u l=180n
Cnw3 nw3 0 2f
CT17 t17 0 0.1f
M39 t17 nw2 vdd vdd pch w=2u l=180n
M40 t17 nq1 vdd vdd pch w=2u l=180n
CT18 t18 0 0.1f
M41 t17 nw2 t18 0 nch w=1u l=180n
M42 t18 nq1 0 0 nch w=1u l=180n
M43 nw4 t17 vdd vdd pch w=2u l=180n
M44 nw4 t17 0 0 nch w=1u l=180n
Cnw4 nw4 0 2f
CT19 t19 0 0.1f
CT20 t20 0 0.1f
CT21 t21 0 0.1f
M45 t19 nq2 vdd vdd pch w=2u l=180n
M46 t19 nw4 vdd vdd pch w=2u l=180n
CT22 t22 0 0.1f
M47 t19 nq2 t22 0 nch w=1u l=180n
M48 t22 nw4 0 0 nch w=1u l=180n
M49 t20 nq2 vdd vdd pch w=2u l=180n
M50 t20 t19 vdd vdd pch w=2u l=180n
CT23 t23 0 0.1f
M51 t20 nq2 t23 0 nch w=1u l=180n
M52 t23 t19 0 0 nch w=1u l=180n
M53 t21 nw4 vdd vdd pch w=2u l=180n
M54 t21 t19 vdd vdd pch w=2u l=180n
CT24 t24 0 0.1f
M55 t21 nw4 t24 0 nch w=1u l=180n
M56 t24 t19 0 0 nch w=1u l=180n
M57 nw5 t20 vdd vdd pch w=2u l=180n
M58 nw5 t21 vdd vdd pch w=2u l=180n
CT25 t25 0 0.1f
M59 nw5 t20 t25 0 nch w=1u l=180n
M60 t25 t21 0 0 nch w=1u l=180n
Cnw5 nw5 0 2f
CT26 t26 0 0.1f
M61 t26 nw4 vdd vdd pch w=2u l=180n
M62 t26 nq2 vdd vdd pch w=2u l=180n
CT27 t27 0 0.1f
M63 t26 nw4 t27 0 nch w=1u l=180n
M64 t27 nq2 0 0 nch w=1u l=180n
M65 nw6 t26 vdd vdd pch w=2u l=180n
M66 nw6 t26 0 0 nch w=1u l=180n
Cnw6 nw6 0 2f
CT28 t28 0 0.1f
CT29 t29 0 0.1f
CT30 t30 0 0.1f
M67 t28 nq3 vdd vdd pch w=2u l=180n
M68 t28 nw6 vdd vdd pch w=2u l=180n
CT31 t31 0 0.1f
M69 t28 nq3 t31 0 nch w=1u l=180n
M70 t31 nw6 0 0 nch w=1u l=180n
M71 t29 nq3 vdd vdd pch w=2u l=180n
M72 t29 t28 vdd vdd pch w=2u l=180n
CT32 t32 0 0.1f
M73 t29 nq3 t32 0 nch w=1u l=180n
M74 t32 t28 0 0 nch w=1u l=180n
M75 t30 nw6 vdd vdd pch w=2u l=180n
M76 t30 t28 vdd vdd pch w=2u l=180n
CT33 t33 0 0.1f
M77 t30 nw6 t33 0 nch w=1u l=180n
M78 t33 t28 0 0 nch w=1u l=180n
M79 nw7 t29 vdd vdd pch w=2u l=180n
M80 nw7 t30 vdd vdd pch w=2u l=180n
CT34 t34 0 0.1f
M81 nw7 t29 t34 0 nch w=1u l=180n
M82 t34 t30 0 0 nch w=1u l=180n
Cnw7 nw7 0 2f
CT35 t35 0 0.1f
M83 t35 nw6 vdd vdd pch w=2u l=180n
M84 t35 nq3 vdd vdd pch w=2u l=180n
CT36 t36 0 0.1f
M85 t35 nw6 t36 0 nch w=1u l=180n
M86 t36 nq3 0 0 nch w=1u l=180n
M87 nw8 t35 vdd vdd pch w=2u l=180n
M88 nw8 t35 0 0 nch w=1u l=180n
Cnw8 nw8 0 2f
CT37 t37 0 0.1f
CT38 t38 0 0.1f
CT39 t39 0 0.1f
M89 t37 nq4 vdd vdd pch w=2u l=180n
M90 t37 nw8 vdd vdd pch w=2u l=180n
CT40 t40 0 0.1f
M91 t37 nq4 t40 0 nch w=1u l=180n
M92 t40 nw8 0 0 nch w=1u l=180n
M93 t38 nq4 vdd vdd pch w=2u l=180n
M94 t38 t37 vdd vdd pch w=2u l=180n
CT41 t41 0 0.1f
M95 t38 nq4 t41 0 nch w=1u l=180n
M96 t41 t37 0 0 nch w=1u l=180n
M97 t39 nw8 vdd vdd pch w=2u l=180n
M98 t39 t37 vdd vdd pch w=2u l=180n
CT42 t42 0 0.1f
M99 t39 nw8 t42 0 nch w=1u l=180n
M100 t42 t37 0 0 nch w=1u l=180n
M101 nw9 t38 vdd vdd pch w=2u l=180n
M102 nw9 t39 vdd vdd pch w=2u l=180n
CT43 t43 0 0.1f
M103 nw9 t38 t43 0 nch w=1u l=180n
M104 t43 t39 0 0 nch w=1u l=180n
Cnw9 nw9 0 2f
CT44 t44 0 0.1f
M105 t44 nw8 vdd vdd pch w=2u l=180n
M106 t44 nq4 vdd vdd pch w=2u l=180n
CT45 t45 0 0.1f
M107 t44 nw8 t45 0 nch w=1u l=180n
M108 t45 nq4 0 0 nch w=1u l=180n
M109 nw10 t44 vdd vdd pch w=2u l=180n
M110 nw10 t44 0 0 nch w=1u l=180n
Cnw10 nw10 0 2f
CT46 t46 0 0.1f
CT47 t47 0 0.1f
CT48 t48 0 0.1f
M111 t46 nq5 vdd vdd pch w=2u l=180n
M112 t46 nw10 vdd vdd pch w=2u l=180n
CT49 t49 0 0.1f
M113 t46 nq5 t49 0 nch w=1u l=180n
M114 t49 nw10 0 0 nch w=1u l=180n
M115 t47 nq5 vdd vdd pch w=2u l=180n
M116 t47 t46 vdd vdd pch w=2u l=180n
CT50 t50 0 0.1f
M117 t47 nq5 t50 0 nch w=1u l=180n
M118 t50 t46 0 0 nch w=1u l=180n
M119 t48 nw10 vdd vdd pch w=2u l=180n
M120 t48 t46 vdd vdd pch w=2u l=180n
CT51 t51 0 0.1f
M121 t48 nw10 t51 0 nch w=1u l=180n
M122 t51 t46 0 0 nch w=1u l=180n
M123 nw11 t47 vdd vdd pch w=2u l=180n
M124 nw11 t48 vdd vdd pch w=2u l=180n
CT52 t52 0 0.1f
M125 nw11 t47 t52 0 nch w=1u l=180n
M126 t52 t48 0 0 nch w=1u l=180n
Cnw11 nw11 0 2f
CT53 t53 0 0.1f
M127 t53 nw10 vdd vdd pch w=2u l=180n
M128 t53 nq5 vdd vdd pch w=2u l=180n
CT54 t54 0 0.1f
M129 t53 nw10 t54 0 nch w=1u l=180n
M130 t54 nq5 0 0 nch w=1u l=180n
M131 nw12 t53 vdd vdd pch w=2u l=180n
M132 nw12 t53 0 0 nch w=1u l=180n
Cnw12 nw12 0 2f
M133 nw13 nq1 vdd vdd pch w=2u l=180n
M134 nw13 nq3 vdd vdd pch w=2u l=180n
CT55 t55 0 0.1f
M135 nw13 nq1 t55 0 nch w=1u l=180n
M136 t55 nq3 0 0 nch w=1u l=180n
Cnw13 nw13 0 2f
M137 nw14 ni2 0 0 nch w=1u l=180n
M138 nw14 nq4 0 0 nch w=1u l=180n
CT56 t56 0 0.1f
M139 t56 ni2 vdd vdd pch w=2u l=180n
M140 nw14 nq4 t56 vdd pch w=2u l=180n
Cnw14 nw14 0 2f
CT57 t57 0 0.1f
M141 t57 nq4 vdd vdd pch w=2u l=180n
M142 t57 nq3 vdd vdd pch w=2u l=180n
CT58 t58 0 0.1f
M143 t57 nq4 t58 0 nch w=1u l=180n
M144 t58 nq3 0 0 nch w=1u l=180n
M145 nw15 t57 vdd vdd pch w=2u l=180n
M146 nw15 t57 0 0 nch w=1u l=180n
Cnw15 nw15 0 2f
CT59 t59 0 0.1f
M147 t59 nw14 0 0 nch w=1u l=180n
M148 t59 nq0 0 0 nch w=1u l=180n
CT60 t60 0 0.1f
M149 t60 nw14 vdd vdd pch w=2u l=180n
M150 t59 nq0 t60 vdd pch w=2u l=180n
M151 nw16 t59 vdd vdd pch w=2u l=180n
M152 nw16 t59 0 0 nch w=1u l=180n
Cnw16 nw16 0 2f
CT61 t61 0 0.1f
CT62 t62 0 0.1f
CT63 t63 0 0.1f
M153 t61 nq3 vdd vdd pch w=2u l=180n
M154 t61 ni2 vdd vdd pch w=2u l=180n
CT64 t64 0 0.1f
M155 t61 nq3 t64 0 nch w=1u l=180n
M156 t64 ni2 0 0 nch w=1u l=180n
M157 t62 nq3 vdd vdd pch w=2u l=180n
M158 t62 t61 vdd vdd pch w=2u l=180n
CT65 t65 0 0.1f
M159 t62 nq3 t65 0 nch w=1u l=180n
M160 t65 t61 0 0 nch w=1u l=180n
M161 t63 ni2 vdd vdd pch w=2u l=180n
M162 t63 t61 vdd vdd pch w=2u l=180n
CT66 t66 0 0.1f
M163 t63 ni2 t66 0 nch w=1u l=180n
M164 t66 t61 0 0 nch w=1u l=180n
M165 nw17 t62 vdd vdd pch w=2u l=180n
M166 nw17 t63 vdd vdd pch w=2u l=180n
CT67 t67 0 0.1f
M167 nw17 t62 t67 0 nch w=1u l=180n
M168 t67 t63 0 0 nch w=1u l=180n
Cnw17 nw17 0 2f
M169 nw18 ni2 vdd vdd pch w=2u l=180n
M170 nw18 nq2 vdd vdd pch w=2u l=180n
CT68 t68 0 0.1f
M171 nw18 ni2 t68 0 nch w=1u l=180n
M172 t68 nq2 0 0 nch w=1u l=180n
Cnw18 nw18 0 2f
M173 nw19 nw17 0 0 nch w=1u l=180n
M174 nw19 nw13 0 0 nch w=1u l=180n
CT69 t69 0 0.1f
M175 t69 nw17 vdd vdd pch w=2u l=180n
M176 nw19 nw13 t69 vdd pch w=2u l=180n
Cnw19 nw19 0 2f
CT70 t70 0 0.1f
M177 t70 nq2 vdd vdd pch w=2u l=180n
M178 t70 nq0 vdd vdd pch w=2u l=180n
CT71 t71 0 0.1f
M179 t70 nq2 t71 0 nch w=1u l=180n
M180 t71 nq0 0 0 nch w=1u l=180n
M181 nw20 t70 vdd vdd pch w=2u l=180n
M182 nw20 t70 0 0 nch w=1u l=180n
Cnw20 nw20 0 2f
CT72 t72 0 0.1f
M183 t72 ni0 0 0 nch w=1u l=180n
M184 t72 ni1 0 0 nch w=1u l=180n
CT73 t73 0 0.1f
M185 t73 ni0 vdd vdd pch w=2u l=180n
M186 t72 ni1 t73 vdd pch w=2u l=180n
M187 nw21 t72 vdd vdd pch w=2u l=180n
M188 nw21 t72 0 0 nch w=1u l=180n
Cnw21 nw21 0 2f
CT74 t74 0 0.1f
CT75 t75 0 0.1f
CT76 t76 0 0.1f
M189 t74 nw14 vdd vdd pch w=2u l=180n
M190 t74 nw16 vdd vdd pch w=2u l=180n
CT77 t77 0 0.1f
M191 t74 nw14 t77 0 nch w=1u l=180n
M192 t77 nw16 0 0 nch w=1u l=180n
M193 t75 nw14 vdd vdd pch w=2u l=180n
M194 t75 t74 vdd vdd pch w=2u l=180n
CT78 t78 0 0.1f
M195 t75 nw14 t78 0 nch w=1u l=180n
M196 t78 t74 0 0 nch w=1u l=180n
M197 t76 nw16 vdd vdd pch w=2u l=180n
M198 t76 t74 vdd vdd pch w=2u l=180n
CT79 t79 0 0.1f
M199 t76 nw16 t79 0 nch w=1u l=180n
M200 t79 t74 0 0 nch w=1u l=180n
M201 nw22 t75 vdd vdd pch w=2u l=180n
M202 nw22 t76 vdd vdd pch w=2u l=180n
CT80 t80 0 0.1f
M203 nw22 t75 t80 0 nch w=1u l=180n
M204 t80 t76 0 0 nch w=1u l=180n
Cnw22 nw22 0 2f
M205 nw23 nw18 vdd vdd pch w=2u l=180n
M206 nw23 nw22 vdd vdd pch w=2u l=180n
CT81 t81 0 0.1f
M207 nw23 nw18 t81 0 nch w=1u l=180n
M208 t81 nw22 0 0 nch w=1u l=180n
Cnw23 nw23 0 2f
M209 nw24 nw22 0 0 nch w=1u l=180n
M210 nw24 nq4 0 0 nch w=1u l=180n
CT82 t82 0 0.1f
M211 t82 nw22 vdd vdd pch w=2u l=180n
M212 nw24 nq4 t82 vdd pch w=2u l=180n
Cnw24 nw24 0 2f
CT83 t83 0 0.1f
M213 t83 nq1 vdd vdd pch w=2u l=180n
M214 t83 nw13 vdd vdd pch w=2u l=180n
CT84 t84 0 0.1f
M215 t83 nq1 t84 0 nch w=1u l=180n
M216 t84 nw13 0 0 nch w=1u l=180n
M217 nw25 t83 vdd vdd pch w=2u l=180n
M218 nw25 t83 0 0 nch w=1u l=180n
Cnw25 nw25 0 2f
CT85 t85 0 0.1f
M219 t85 nq4 0 0 nch w=1u l=180n
M220 t85 nw18 0 0 nch w=1u l=180n
CT86 t86 0 0.1f
M221 t86 nq4 vdd vdd pch w=2u l=180n
M222 t85 nw18 t86 vdd pch w=2u l=180n
M223 nw26 t85 vdd vdd pch w=2u l=180n
M224 nw26 t85 0 0 nch w=1u l=180n
Cnw26 nw26 0 2f
CT87 t87 0 0.1f
CT88 t88 0 0.1f
CT89 t89 0 0.1f
M225 t87 ni1 vdd vdd pch w=2u l=180n
M226 t87 nw23 vdd vdd pch w=2u l=180n
CT90 t90 0 0.1f
M227 t87 ni1 t90 0 nch w=1u l=180n
M228 t90 nw23 0 0 nch w=1u l=180n
M229 t88 ni1 vdd vdd pch w=2u l=180n
M230 t88 t87 vdd vdd pch w=2u l=180n
CT91 t91 0 0.1f
M231 t88 ni1 t91 0 nch w=1u l=180n
M232 t91 t87 0 0 nch w=1u l=180n
M233 t89 nw23 vdd vdd pch w=2u l=180n
M234 t89 t87 vdd vdd pch w=2u l=180n
CT92 t92 0 0.1f
M235 t89 nw23 t92 0 nch w=1u l=180n
M236 t92 t87 0 0 nch w=1u l=180n
M237 nw27 t88 vdd vdd pch w=2u l=180n
M238 nw27 t89 vdd vdd pch w=2u l=180n
CT93 t93 0 0.1f
M239 nw27 t88 t93 0 nch w=1u l=180n
M240 t93 t89 0 0 nch w=1u l=180n
Cnw27 nw27 0 2f
M241 nw28 nw14 vdd vdd pch w=2u l=180n
M242 nw28 nq0 vdd vdd pch w=2u l=180n
CT94 t94 0 0.1f
M243 nw28 nw14 t94 0 nch w=1u l=180n
M244 t94 nq0 0 0 nch w=1u l=180n
Cnw28 nw28 0 2f
M245 nw29 nw17 0 0 nch w=1u l=180n
M246 nw29 nq4 0 0 nch w=1u l=180n
CT95 t95 0 0.1f
M247 t95 nw17 vdd vdd pch w=2u l=180n
M248 nw29 nq4 t95 vdd pch w=2u l=180n
Cnw29 nw29 0 2f
CT96 t96 0 0.1f
M249 t96 nw20 vdd vdd pch w=2u l=180n
M250 t96 ni2 vdd vdd pch w=2u l=180n
CT97 t97 0 0.1f
M251 t96 nw20 t97 0 nch w=1u l=180n
M252 t97 ni2 0 0 nch w=1u l=180n
M253 nw30 t96 vdd vdd pch w=2u l=180n
M254 nw30 t96 0 0 nch w=1u l=180n
Cnw30 nw30 0 2f
CT98 t98 0 0.1f
M255 t98 nw23 0 0 nch w=1u l=180n
M256 t98 nw16 0 0 nch w=1u l=180n
CT99 t99 0 0.1f
M257 t99 nw23 vdd vdd pch w=2u l=180n
M258 t98 nw16 t99 vdd pch w=2u l=180n
M259 nw31 t98 vdd vdd pch w=2u l=180n
M260 nw31 t98 0 0 nch w=1u l=180n
Cnw31 nw31 0 2f
CT100 t100 0 0.1f
CT101 t101 0 0.1f
CT102 t102 0 0.1f
M261 t100 nw26 vdd vdd pch w=2u l=180n
M262 t100 nw20 vdd vdd pch w=2u l=180n
CT103 t103 0 0.1f
M263 t100 nw26 t103 0 nch w=1u l=180n
M264 t103 nw20 0 0 nch w=1u l=180n
M265 t101 nw26 vdd vdd pch w=2u l=180n
M266 t101 t100 vdd vdd pch w=2u l=180n
CT104 t104 0 0.1f
M267 t101 nw26 t104 0 nch w=1u l=180n
M268 t104 t100 0 0 nch w=1u l=180n
M269 t102 nw20 vdd vdd pch w=2u l=180n
M270 t102 t100 vdd vdd pch w=2u l=180n
CT105 t105 0 0.1f
M271 t102 nw20 t105 0 nch w=1u l=180n
M272 t105 t100 0 0 nch w=1u l=180n
M273 nw32 t101 vdd vdd pch w=2u l=180n
M274 nw32 t102 vdd vdd pch w=2u l=180n
CT106 t106 0 0.1f
M275 nw32 t101 t106 0 nch w=1u l=180n
M276 t106 t102 0 0 nch w=1u l=180n
Cnw32 nw32 0 2f
M277 nw33 nw29 vdd vdd pch w=2u l=180n
M278 nw33 nw24 vdd vdd pch w=2u l=180n
CT107 t107 0 0.1f
M279 nw33 nw29 t107 0 nch w=1u l=180n
M280 t107 nw24 0 0 nch w=1u l=180n
Cnw33 nw33 0 2f
M281 nw34 nw32 0 0 nch w=1u l=180n
M282 nw34 nw28 0 0 nch w=1u l=180n
CT108 t108 0 0.1f
M283 t108 nw32 vdd vdd pch w=2u l=180n
M284 nw34 nw28 t108 vdd pch w=2u l=180n
Cnw34 nw34 0 2f
CT109 t109 0 0.1f
M285 t109 nq0 vdd vdd pch w=2u l=180n
M286 t109 nw32 vdd vdd pch w=2u l=180n
CT110 t110 0 0.1f
M287 t109 nq0 t110 0 nch w=1u l=180n
M288 t110 nw32 0 0 nch w=1u l=180n
M289 nw35 t109 vdd vdd pch w=2u l=180n
M290 nw35 t109 0 0 nch w=1u l=180n
Cnw35 nw35 0 2f
CT111 t111 0 0.1f
M291 t111 nq2 0 0 nch w=1u l=180n
M292 t111 nq0 0 0 nch w=1u l=180n
CT112 t112 0 0.1f
M293 t112 nq2 vdd vdd pch w=2u l=180n
M294 t111 nq0 t112 vdd pch w=2u l=180n
M295 nw36 t111 vdd vdd pch w=2u l=180n
M296 nw36 t111 0 0 nch w=1u l=180n
Cnw36 nw36 0 2f
CT113 t113 0 0.1f
CT114 t114 0 0.1f
CT115 t115 0 0.1f
M297 t113 nq4 vdd vdd pch w=2u l=180n
M298 t113 nq3 vdd vdd pch w=2u l=180n
CT116 t116 0 0.1f
M299 t113 nq4 t116 0 nch w=1u l=180n
M300 t116 nq3 0 0 nch w=1u l=180n
M301 t114 nq4 vdd vdd pch w=2u l=180n
M302 t114 t113 vdd vdd pch w=2u l=180n
CT117 t117 0 0.1f
M303 t114 nq4 t117 0 nch w=1u l=180n
M304 t117 t113 0 0 nch w=1u l=180n
M305 t115 nq3 vdd vdd pch w=2u l=180n
M306 t115 t113 vdd vdd pch w=2u l=180n
CT118 t118 0 0.1f
M307 t115 nq3 t118 0 nch w=1u l=180n
M308 t118 t113 0 0 nch w=1u l=180n
M309 nw37 t114 vdd vdd pch w=2u l=180n
M310 nw37 t115 vdd vdd pch w=2u l=180n
CT119 t119 0 0.1f
M311 nw37 t114 t119 0 nch w=1u l=180n
M312 t119 t115 0 0 nch w=1u l=180n
Cnw37 nw37 0 2f
M313 nw38 ni0 vdd vdd pch w=2u l=180n
M314 nw38 nw28 vdd vdd pch w=2u l=180n
CT120 t120 0 0.1f
M315 nw38 ni0 t120 0 nch w=1u l=180n
M316 t120 nw28 0 0 nch w=1u l=180n
Cnw38 nw38 0 2f
M317 nw39 ni2 0 0 nch w=1u l=180n
M318 nw39 nw13 0 0 nch w=1u l=180n
CT121 t121 0 0.1f
M319 t121 ni2 vdd vdd pch w=2u l=180n
M320 nw39 nw13 t121 vdd pch w=2u l=180n
Cnw39 nw39 0 2f
CT122 t122 0 0.1f
M321 t122 nw14 vdd vdd pch w=2u l=180n
M322 t122 nw16 vdd vdd pch w=2u l=180n
CT123 t123 0 0.1f
M323 t122 nw14 t123 0 nch w=1u l=180n
M324 t123 nw16 0 0 nch w=1u l=180n
M325 nw40 t122 vdd vdd pch w=2u l=180n
M326 nw40 t122 0 0 nch w=1u l=180n
Cnw40 nw40 0 2f
CT124 t124 0 0.1f
M327 t124 nw16 0 0 nch w=1u l=180n
M328 t124 nw19 0 0 nch w=1u l=180n
CT125 t125 0 0.1f
M329 t125 nw16 vdd vdd pch w=2u l=180n
M330 t124 nw19 t125 vdd pch w=2u l=180n
M331 nw41 t124 vdd vdd pch w=2u l=180n
M332 nw41 t124 0 0 nch w=1u l=180n
Cnw41 nw41 0 2f
CT126 t126 0 0.1f
CT127 t127 0 0.1f
CT128 t128 0 0.1f
M333 t126 nw18 vdd vdd pch w=2u l=180n
M334 t126 nw22 vdd vdd pch w=2u l=180n
CT129 t129 0 0.1f
M335 t126 nw18 t129 0 nch w=1u l=180n
M336 t129 nw22 0 0 nch w=1u l=180n
M337 t127 nw18 vdd vdd pch w=2u l=180n
M338 t127 t126 vdd vdd pch w=2u l=180n
CT130 t130 0 0.1f
M339 t127 nw18 t130 0 nch w=1u l=180n
M340 t130 t126 0 0 nch w=1u l=180n
M341 t128 nw22 vdd vdd pch w=2u l=180n
M342 t128 t126 vdd vdd pch w=2u l=180n
CT131 t131 0 0.1f
M343 t128 nw22 t131 0 nch w=1u l=180n
M344 t131 t126 0 0 nch w=1u l=180n
M345 nw42 t127 vdd vdd pch w=2u l=180n
M346 nw42 t128 vdd vdd pch w=2u l=180n
CT132 t132 0 0.1f
M347 nw42 t127 t132 0 nch w=1u l=180n
M348 t132 t128 0 0 nch w=1u l=180n
Cnw42 nw42 0 2f
M349 nw43 nw20 vdd vdd pch w=2u l=180n
M350 nw43 nw25 vdd vdd pch w=2u l=180n
CT133 t133 0 0.1f
M351 nw43 nw20 t133 0 nch w=1u l=180n
M352 t133 nw25 0 0 nch w=1u l=180n
Cnw43 nw43 0 2f
M353 nw44 nw22 0 0 nch w=1u l=180n
M354 nw44 nw28 0 0 nch w=1u l=180n
CT134 t134 0 0.1f
M355 t134 nw22 vdd vdd pch w=2u l=180n
M356 nw44 nw28 t134 vdd pch w=2u l=180n
Cnw44 nw44 0 2f
CT135 t135 0 0.1f
M357 t135 nw24 vdd vdd pch w=2u l=180n
M358 t135 nw31 vdd vdd pch w=2u l=180n
CT136 t136 0 0.1f
M359 t135 nw24 t136 0 nch w=1u l=180n
M360 t136 nw31 0 0 nch w=1u l=180n
M361 nw45 t135 vdd vdd pch w=2u l=180n
M362 nw45 t135 0 0 nch w=1u l=180n
Cnw45 nw45 0 2f
CT137 t137 0 0.1f
M363 t137 nw26 0 0 nch w=1u l=180n
M364 t137 nw34 0 0 nch w=1u l=180n
CT138 t138 0 0.1f
M365 t138 nw26 vdd vdd pch w=2u l=180n
M366 t137 nw34 t138 vdd pch w=2u l=180n
M367 nw46 t137 vdd vdd pch w=2u l=180n
M368 nw46 t137 0 0 nch w=1u l=180n
Cnw46 nw46 0 2f
CT139 t139 0 0.1f
CT140 t140 0 0.1f
CT141 t141 0 0.1f
M369 t139 nw28 vdd vdd pch w=2u l=180n
M370 t139 nw37 vdd vdd pch w=2u l=180n
CT142 t142 0 0.1f
M371 t139 nw28 t142 0 nch w=1u l=180n
M372 t142 nw37 0 0 nch w=1u l=180n
M373 t140 nw28 vdd vdd pch w=2u l=180n
M374 t140 t139 vdd vdd pch w=2u l=180n
CT143 t143 0 0.1f
M375 t140 nw28 t143 0 nch w=1u l=180n
M376 t143 t139 0 0 nch w=1u l=180n
M377 t141 nw37 vdd vdd pch w=2u l=180n
M378 t141 t139 vdd vdd pch w=2u l=180n
CT144 t144 0 0.1f
M379 t141 nw37 t144 0 nch w=1u l=180n
M380 t144 t139 0 0 nch w=1u l=180n
M381 nw47 t140 vdd vdd pch w=2u l=180n
M382 nw47 t141 vdd vdd pch w=2u l=180n
CT145 t145 0 0.1f
M383 nw47 t140 t145 0 nch w=1u l=180n
M384 t145 t141 0 0 nch w=1u l=180n
Cnw47 nw47 0 2f
M385 nw48 nw30 vdd vdd pch w=2u l=180n
M386 nw48 nw40 vdd vdd pch w=2u l=180n
CT146 t146 0 0.1f
M387 nw48 nw30 t146 0 nch w=1u l=180n
M388 t146 nw40 0 0 nch w=1u l=180n
Cnw48 nw48 0 2f
M389 nw49 nw32 0 0 nch w=1u l=180n
M390 nw49 nw43 0 0 nch w=1u l=180n
CT147 t147 0 0.1f
M391 t147 nw32 vdd vdd pch w=2u l=180n
M392 nw49 nw43 t147 vdd pch w=2u l=180n
Cnw49 nw49 0 2f
CT148 t148 0 0.1f
M393 t148 nw34 vdd vdd pch w=2u l=180n
M394 t148 nw46 vdd vdd pch w=2u l=180n
CT149 t149 0 0.1f
M395 t148 nw34 t149 0 nch w=1u l=180n
M396 t149 nw46 0 0 nch w=1u l=180n
M397 nw50 t148 vdd vdd pch w=2u l=180n
M398 nw50 t148 0 0 nch w=1u l=180n
Cnw50 nw50 0 2f
CT150 t150 0 0.1f
M399 t150 nw36 0 0 nch w=1u l=180n
M400 t150 nw49 0 0 nch w=1u l=180n
CT151 t151 0 0.1f
M401 t151 nw36 vdd vdd pch w=2u l=180n
M402 t150 nw49 t151 vdd pch w=2u l=180n
M403 nw51 t150 vdd vdd pch w=2u l=180n
M404 nw51 t150 0 0 nch w=1u l=180n
Cnw51 nw51 0 2f
CT152 t152 0 0.1f
CT153 t153 0 0.1f
CT154 t154 0 0.1f
M405 t152 nw38 vdd vdd pch w=2u l=180n
M406 t152 nq0 vdd vdd pch w=2u l=180n
CT155 t155 0 0.1f
M407 t152 nw38 t155 0 nch w=1u l=180n
M408 t155 nq0 0 0 nch w=1u l=180n
M409 t153 nw38 vdd vdd pch w=2u l=180n
M410 t153 t152 vdd vdd pch w=2u l=180n
CT156 t156 0 0.1f
M411 t153 nw38 t156 0 nch w=1u l=180n
M412 t156 t152 0 0 nch w=1u l=180n
M413 t154 nq0 vdd vdd pch w=2u l=180n
M414 t154 t152 vdd vdd pch w=2u l=180n
CT157 t157 0 0.1f
M415 t154 nq0 t157 0 nch w=1u l=180n
M416 t157 t152 0 0 nch w=1u l=180n
M417 nw52 t153 vdd vdd pch w=2u l=180n
M418 nw52 t154 vdd vdd pch w=2u l=180n
CT158 t158 0 0.1f
M419 nw52 t153 t158 0 nch w=1u l=180n
M420 t158 t154 0 0 nch w=1u l=180n
Cnw52 nw52 0 2f
M421 nw53 nw40 vdd vdd pch w=2u l=180n
M422 nw53 nq2 vdd vdd pch w=2u l=180n
CT159 t159 0 0.1f
M423 nw53 nw40 t159 0 nch w=1u l=180n
M424 t159 nq2 0 0 nch w=1u l=180n
Cnw53 nw53 0 2f
M425 nw54 nw42 0 0 nch w=1u l=180n
M426 nw54 nq4 0 0 nch w=1u l=180n
CT160 t160 0 0.1f
M427 t160 nw42 vdd vdd pch w=2u l=180n
M428 nw54 nq4 t160 vdd pch w=2u l=180n
Cnw54 nw54 0 2f
CT161 t161 0 0.1f
M429 t161 nw44 vdd vdd pch w=2u l=180n
M430 t161 ni0 vdd vdd pch w=2u l=180n
CT162 t162 0 0.1f
M431 t161 nw44 t162 0 nch w=1u l=180n
M432 t162 ni0 0 0 nch w=1u l=180n
M433 nw55 t161 vdd vdd pch w=2u l=180n
M434 nw55 t161 0 0 nch w=1u l=180n
Cnw55 nw55 0 2f
CT163 t163 0 0.1f
M435 t163 nw46 0 0 nch w=1u l=180n
M436 t163 ni2 0 0 nch w=1u l=180n
CT164 t164 0 0.1f
M437 t164 nw46 vdd vdd pch w=2u l=180n
M438 t163 ni2 t164 vdd pch w=2u l=180n
M439 nw56 t163 vdd vdd pch w=2u l=180n
M440 nw56 t163 0 0 nch w=1u l=180n
Cnw56 nw56 0 2f
CT165 t165 0 0.1f
CT166 t166 0 0.1f
CT167 t167 0 0.1f
M441 t165 nw48 vdd vdd pch w=2u l=180n
M442 t165 nw14 vdd vdd pch w=2u l=180n
CT168 t168 0 0.1f
M443 t165 nw48 t168 0 nch w=1u l=180n
M444 t168 nw14 0 0 nch w=1u l=180n
M445 t166 nw48 vdd vdd pch w=2u l=180n
M446 t166 t165 vdd vdd pch w=2u l=180n
CT169 t169 0 0.1f
M447 t166 nw48 t169 0 nch w=1u l=180n
M448 t169 t165 0 0 nch w=1u l=180n
M449 t167 nw14 vdd vdd pch w=2u l=180n
M450 t167 t165 vdd vdd pch w=2u l=180n
CT170 t170 0 0.1f
M451 t167 nw14 t170 0 nch w=1u l=180n
M452 t170 t165 0 0 nch w=1u l=180n
M453 nw57 t166 vdd vdd pch w=2u l=180n
M454 nw57 t167 vdd vdd pch w=2u l=180n
CT171 t171 0 0.1f
M455 nw57 t166 t171 0 nch w=1u l=180n
M456 t171 t167 0 0 nch w=1u l=180n
Cnw57 nw57 0 2f
M457 nw58 nw50 vdd vdd pch w=2u l=180n
M458 nw58 nw16 vdd vdd pch w=2u l=180n
CT172 t172 0 0.1f
M459 nw58 nw50 t172 0 nch w=1u l=180n
M460 t172 nw16 0 0 nch w=1u l=180n
Cnw58 nw58 0 2f
M461 nw59 nw52 0 0 nch w=1u l=180n
M462 nw59 nw18 0 0 nch w=1u l=180n
CT173 t173 0 0.1f
M463 t173 nw52 vdd vdd pch w=2u l=180n
M464 nw59 nw18 t173 vdd pch w=2u l=180n
Cnw59 nw59 0 2f
CT174 t174 0 0.1f
M465 t174 nw54 vdd vdd pch w=2u l=180n
M466 t174 nw20 vdd vdd pch w=2u l=180n
CT175 t175 0 0.1f
M467 t174 nw54 t175 0 nch w=1u l=180n
M468 t175 nw20 0 0 nch w=1u l=180n
M469 nw60 t174 vdd vdd pch w=2u l=180n
M470 nw60 t174 0 0 nch w=1u l=180n
Cnw60 nw60 0 2f
CT176 t176 0 0.1f
M471 t176 nw56 0 0 nch w=1u l=180n
M472 t176 nw22 0 0 nch w=1u l=180n
CT177 t177 0 0.1f
M473 t177 nw56 vdd vdd pch w=2u l=180n
M474 t176 nw22 t177 vdd pch w=2u l=180n
M475 nw61 t176 vdd vdd pch w=2u l=180n
M476 nw61 t176 0 0 nch w=1u l=180n
Cnw61 nw61 0 2f
CT178 t178 0 0.1f
CT179 t179 0 0.1f
CT180 t180 0 0.1f
M477 t178 nw58 vdd vdd pch w=2u l=180n
M478 t178 nw24 vdd vdd pch w=2u l=180n
CT181 t181 0 0.1f
M479 t178 nw58 t181 0 nch w=1u l=180n
M480 t181 nw24 0 0 nch w=1u l=180n
M481 t179 nw58 vdd vdd pch w=2u l=180n
M482 t179 t178 vdd vdd pch w=2u l=180n
CT182 t182 0 0.1f
M483 t179 nw58 t182 0 nch w=1u l=180n
M484 t182 t178 0 0 nch w=1u l=180n
M485 t180 nw24 vdd vdd pch w=2u l=180n
M486 t180 t178 vdd vdd pch w=2u l=180n
CT183 t183 0 0.1f
M487 t180 nw24 t183 0 nch w=1u l=180n
M488 t183 t178 0 0 nch w=1u l=180n
M489 nw62 t179 vdd vdd pch w=2u l=180n
M490 nw62 t180 vdd vdd pch w=2u l=180n
CT184 t184 0 0.1f
M491 nw62 t179 t184 0 nch w=1u l=180n
M492 t184 t180 0 0 nch w=1u l=180n
Cnw62 nw62 0 2f
M493 nw63 nw60 vdd vdd pch w=2u l=180n
M494 nw63 nw26 vdd vdd pch w=2u l=180n
CT185 t185 0 0.1f
M495 nw63 nw60 t185 0 nch w=1u l=180n
M496 t185 nw26 0 0 nch w=1u l=180n
Cnw63 nw63 0 2f
M497 nw64 nw62 0 0 nch w=1u l=180n
M498 nw64 nw28 0 0 nch w=1u l=180n
CT186 t186 0 0.1f
M499 t186 nw62 vdd vdd pch w=2u l=180n
M500 nw64 nw28 t186 vdd pch w=2u l=180n
Cnw64 nw64 0 2f
CT187 t187 0 0.1f
M501 t187 nw64 vdd vdd pch w=2u l=180n
M502 t187 nw30 vdd vdd pch w=2u l=180n
CT188 t188 0 0.1f
M503 t187 nw64 t188 0 nch w=1u l=180n
M504 t188 nw30 0 0 nch w=1u l=180n
M505 nw65 t187 vdd vdd pch w=2u l=180n
M506 nw65 t187 0 0 nch w=1u l=180n
Cnw65 nw65 0 2f
CT189 t189 0 0.1f
M507 t189 nq0 0 0 nch w=1u l=180n
M508 t189 nw32 0 0 nch w=1u l=180n
CT190 t190 0 0.1f
M509 t190 nq0 vdd vdd pch w=2u l=180n
M510 t189 nw32 t190 vdd pch w=2u l=180n
M511 nw66 t189 vdd vdd pch w=2u l=180n
M512 nw66 t189 0 0 nch w=1u l=180n
Cnw66 nw66 0 2f
CT191 t191 0 0.1f
CT192 t192 0 0.1f
CT193 t193 0 0.1f
M513 t191 nq1 vdd vdd pch w=2u l=180n
M514 t191 nw34 vdd vdd pch w=2u l=180n
CT194 t194 0 0.1f
M515 t191 nq1 t194 0 nch w=1u l=180n
M516 t194 nw34 0 0 nch w=1u l=180n
M517 t192 nq1 vdd vdd pch w=2u l=180n
M518 t192 t191 vdd vdd pch w=2u l=180n
CT195 t195 0 0.1f
M519 t192 nq1 t195 0 nch w=1u l=180n
M520 t195 t191 0 0 nch w=1u l=180n
M521 t193 nw34 vdd vdd pch w=2u l=180n
M522 t193 t191 vdd vdd pch w=2u l=180n
CT196 t196 0 0.1f
M523 t193 nw34 t196 0 nch w=1u l=180n
M524 t196 t191 0 0 nch w=1u l=180n
M525 nw67 t192 vdd vdd pch w=2u l=180n
M526 nw67 t193 vdd vdd pch w=2u l=180n
CT197 t197 0 0.1f
M527 nw67 t192 t197 0 nch w=1u l=180n
M528 t197 t193 0 0 nch w=1u l=180n
Cnw67 nw67 0 2f
M529 nw68 nq2 vdd vdd pch w=2u l=180n
M530 nw68 nw36 vdd vdd pch w=2u l=180n
CT198 t198 0 0.1f
M531 nw68 nq2 t198 0 nch w=1u l=180n
M532 t198 nw36 0 0 nch w=1u l=180n
Cnw68 nw68 0 2f
M533 nw69 nq3 0 0 nch w=1u l=180n
M534 nw69 nw38 0 0 nch w=1u l=180n
CT199 t199 0 0.1f
M535 t199 nq3 vdd vdd pch w=2u l=180n
M536 nw69 nw38 t199 vdd pch w=2u l=180n
Cnw69 nw69 0 2f
CT200 t200 0 0.1f
M537 t200 nq4 vdd vdd pch w=2u l=180n
M538 t200 nw40 vdd vdd pch w=2u l=180n
CT201 t201 0 0.1f
M539 t200 nq4 t201 0 nch w=1u l=180n
M540 t201 nw40 0 0 nch w=1u l=180n
M541 nw70 t200 vdd vdd pch w=2u l=180n
M542 nw70 t200 0 0 nch w=1u l=180n
Cnw70 nw70 0 2f
CT202 t202 0 0.1f
M543 t202 nq5 0 0 nch w=1u l=180n
M544 t202 nw42 0 0 nch w=1u l=180n
CT203 t203 0 0.1f
M545 t203 nq5 vdd vdd pch w=2u l=180n
M546 t202 nw42 t203 vdd pch w=2u l=180n
M547 nw71 t202 vdd vdd pch w=2u l=180n
M548 nw71 t202 0 0 nch w=1u l=180n
Cnw71 nw71 0 2f
CT204 t204 0 0.1f
CT205 t205 0 0.1f
CT206 t206 0 0.1f
M549 t204 ni0 vdd vdd pch w=2u l=180n
M550 t204 nw44 vdd vdd pch w=2u l=180n
CT207 t207 0 0.1f
M551 t204 ni0 t207 0 nch w=1u l=180n
M552 t207 nw44 0 0 nch w=1u l=180n
M553 t205 ni0 vdd vdd pch w=2u l=180n
M554 t205 t204 vdd vdd pch w=2u l=180n
CT208 t208 0 0.1f
M555 t205 ni0 t208 0 nch w=1u l=180n
M556 t208 t204 0 0 nch w=1u l=180n
M557 t206 nw44 vdd vdd pch w=2u l=180n
M558 t206 t204 vdd vdd pch w=2u l=180n
CT209 t209 0 0.1f
M559 t206 nw44 t209 0 nch w=1u l=180n
M560 t209 t204 0 0 nch w=1u l=180n
M561 nw72 t205 vdd vdd pch w=2u l=180n
M562 nw72 t206 vdd vdd pch w=2u l=180n
CT210 t210 0 0.1f
M563 nw72 t205 t210 0 nch w=1u l=180n
M564 t210 t206 0 0 nch w=1u l=180n
Cnw72 nw72 0 2f
M565 nw73 ni1 vdd vdd pch w=2u l=180n
M566 nw73 nw46 vdd vdd pch w=2u l=180n
CT211 t211 0 0.1f
M567 nw73 ni1 t211 0 nch w=1u l=180n
M568 t211 nw46 0 0 nch w=1u l=180n
Cnw73 nw73 0 2f
M569 nw74 ni2 0 0 nch w=1u l=180n
M570 nw74 nw48 0 0 nch w=1u l=180n
CT212 t212 0 0.1f
M571 t212 ni2 vdd vdd pch w=2u l=180n
M572 nw74 nw48 t212 vdd pch w=2u l=180n
Cnw74 nw74 0 2f
CT213 t213 0 0.1f
M573 t213 nw13 vdd vdd pch w=2u l=180n
M574 t213 nw50 vdd vdd pch w=2u l=180n
CT214 t214 0 0.1f
M575 t213 nw13 t214 0 nch w=1u l=180n
M576 t214 nw50 0 0 nch w=1u l=180n
M577 nw75 t213 vdd vdd pch w=2u l=180n
M578 nw75 t213 0 0 nch w=1u l=180n
Cnw75 nw75 0 2f
CT215 t215 0 0.1f
M579 t215 nw14 0 0 nch w=1u l=180n
M580 t215 nw52 0 0 nch w=1u l=180n
CT216 t216 0 0.1f
M581 t216 nw14 vdd vdd pch w=2u l=180n
M582 t215 nw52 t216 vdd pch w=2u l=180n
M583 nw76 t215 vdd vdd pch w=2u l=180n
M584 nw76 t215 0 0 nch w=1u l=180n
Cnw76 nw76 0 2f
CT217 t217 0 0.1f
CT218 t218 0 0.1f
CT219 t219 0 0.1f
M585 t217 nw15 vdd vdd pch w=2u l=180n
M586 t217 nw54 vdd vdd pch w=2u l=180n
CT220 t220 0 0.1f
M587 t217 nw15 t220 0 nch w=1u l=180n
M588 t220 nw54 0 0 nch w=1u l=180n
M589 t218 nw15 vdd vdd pch w=2u l=180n
M590 t218 t217 vdd vdd pch w=2u l=180n
CT221 t221 0 0.1f
M591 t218 nw15 t221 0 nch w=1u l=180n
M592 t221 t217 0 0 nch w=1u l=180n
M593 t219 nw54 vdd vdd pch w=2u l=180n
M594 t219 t217 vdd vdd pch w=2u l=180n
CT222 t222 0 0.1f
M595 t219 nw54 t222 0 nch w=1u l=180n
M596 t222 t217 0 0 nch w=1u l=180n
M597 nw77 t218 vdd vdd pch w=2u l=180n
M598 nw77 t219 vdd vdd pch w=2u l=180n
CT223 t223 0 0.1f
M599 nw77 t218 t223 0 nch w=1u l=180n
M600 t223 t219 0 0 nch w=1u l=180n
Cnw77 nw77 0 2f
M601 nw78 nw16 vdd vdd pch w=2u l=180n
M602 nw78 nw56 vdd vdd pch w=2u l=180n
CT224 t224 0 0.1f
M603 nw78 nw16 t224 0 nch w=1u l=180n
M604 t224 nw56 0 0 nch w=1u l=180n
Cnw78 nw78 0 2f
M605 nw79 nw17 0 0 nch w=1u l=180n
M606 nw79 nw58 0 0 nch w=1u l=180n
CT225 t225 0 0.1f
M607 t225 nw17 vdd vdd pch w=2u l=180n
M608 nw79 nw58 t225 vdd pch w=2u l=180n
Cnw79 nw79 0 2f
CT226 t226 0 0.1f
M609 t226 nw18 vdd vdd pch w=2u l=180n
M610 t226 nw60 vdd vdd pch w=2u l=180n
CT227 t227 0 0.1f
M611 t226 nw18 t227 0 nch w=1u l=180n
M612 t227 nw60 0 0 nch w=1u l=180n
M613 nw80 t226 vdd vdd pch w=2u l=180n
M614 nw80 t226 0 0 nch w=1u l=180n
Cnw80 nw80 0 2f
CT228 t228 0 0.1f
M615 t228 nw19 0 0 nch w=1u l=180n
M616 t228 nw62 0 0 nch w=1u l=180n
CT229 t229 0 0.1f
M617 t229 nw19 vdd vdd pch w=2u l=180n
M618 t228 nw62 t229 vdd pch w=2u l=180n
M619 nw81 t228 vdd vdd pch w=2u l=180n
M620 nw81 t228 0 0 nch w=1u l=180n
Cnw81 nw81 0 2f
CT230 t230 0 0.1f
CT231 t231 0 0.1f
CT232 t232 0 0.1f
M621 t230 nw20 vdd vdd pch w=2u l=180n
M622 t230 nw64 vdd vdd pch w=2u l=180n
CT233 t233 0 0.1f
M623 t230 nw20 t233 0 nch w=1u l=180n
M624 t233 nw64 0 0 nch w=1u l=180n
M625 t231 nw20 vdd vdd pch w=2u l=180n
M626 t231 t230 vdd vdd pch w=2u l=180n
CT234 t234 0 0.1f
M627 t231 nw20 t234 0 nch w=1u l=180n
M628 t234 t230 0 0 nch w=1u l=180n
M629 t232 nw64 vdd vdd pch w=2u l=180n
M630 t232 t230 vdd vdd pch w=2u l=180n
CT235 t235 0 0.1f
M631 t232 nw64 t235 0 nch w=1u l=180n
M632 t235 t230 0 0 nch w=1u l=180n
M633 nw82 t231 vdd vdd pch w=2u l=180n
M634 nw82 t232 vdd vdd pch w=2u l=180n
CT236 t236 0 0.1f
M635 nw82 t231 t236 0 nch w=1u l=180n
M636 t236 t232 0 0 nch w=1u l=180n
Cnw82 nw82 0 2f
M637 nw83 nw21 vdd vdd pch w=2u l=180n
M638 nw83 nw66 vdd vdd pch w=2u l=180n
CT237 t237 0 0.1f
M639 nw83 nw21 t237 0 nch w=1u l=180n
M640 t237 nw66 0 0 nch w=1u l=180n
Cnw83 nw83 0 2f
M641 nw84 nw22 0 0 nch w=1u l=180n
M642 nw84 nw68 0 0 nch w=1u l=180n
CT238 t238 0 0.1f
M643 t238 nw22 vdd vdd pch w=2u l=180n
M644 nw84 nw68 t238 vdd pch w=2u l=180n
Cnw84 nw84 0 2f
CT239 t239 0 0.1f
M645 t239 nw23 vdd vdd pch w=2u l=180n
M646 t239 nw70 vdd vdd pch w=2u l=180n
CT240 t240 0 0.1f
M647 t239 nw23 t240 0 nch w=1u l=180n
M648 t240 nw70 0 0 nch w=1u l=180n
M649 nw85 t239 vdd vdd pch w=2u l=180n
M650 nw85 t239 0 0 nch w=1u l=180n
Cnw85 nw85 0 2f
CT241 t241 0 0.1f
M651 t241 nw24 0 0 nch w=1u l=180n
M652 t241 nw72 0 0 nch w=1u l=180n
CT242 t242 0 0.1f
M653 t242 nw24 vdd vdd pch w=2u l=180n
M654 t241 nw72 t242 vdd pch w=2u l=180n
M655 nw86 t241 vdd vdd pch w=2u l=180n
M656 nw86 t241 0 0 nch w=1u l=180n
Cnw86 nw86 0 2f
CT243 t243 0 0.1f
CT244 t244 0 0.1f
CT245 t245 0 0.1f
M657 t243 nw25 vdd vdd pch w=2u l=180n
M658 t243 nw74 vdd vdd pch w=2u l=180n
CT246 t246 0 0.1f
M659 t243 nw25 t246 0 nch w=1u l=180n
M660 t246 nw74 0 0 nch w=1u l=180n
M661 t244 nw25 vdd vdd pch w=2u l=180n
M662 t244 t243 vdd vdd pch w=2u l=180n
CT247 t247 0 0.1f
M663 t244 nw25 t247 0 nch w=1u l=180n
M664 t247 t243 0 0 nch w=1u l=180n
M665 t245 nw74 vdd vdd pch w=2u l=180n
M666 t245 t243 vdd vdd pch w=2u l=180n
CT248 t248 0 0.1f
M667 t245 nw74 t248 0 nch w=1u l=180n
M668 t248 t243 0 0 nch w=1u l=180n
M669 nw87 t244 vdd vdd pch w=2u l=180n
M670 nw87 t245 vdd vdd pch w=2u l=180n
CT249 t249 0 0.1f
M671 nw87 t244 t249 0 nch w=1u l=180n
M672 t249 t245 0 0 nch w=1u l=180n
Cnw87 nw87 0 2f
M673 nw88 nw26 vdd vdd pch w=2u l=180n
M674 nw88 nw76 vdd vdd pch w=2u l=180n
CT250 t250 0 0.1f
M675 nw88 nw26 t250 0 nch w=1u l=180n
M676 t250 nw76 0 0 nch w=1u l=180n
Cnw88 nw88 0 2f
M677 nw89 nw27 0 0 nch w=1u l=180n
M678 nw89 nw78 0 0 nch w=1u l=180n
CT251 t251 0 0.1f
M679 t251 nw27 vdd vdd pch w=2u l=180n
M680 nw89 nw78 t251 vdd pch w=2u l=180n
Cnw89 nw89 0 2f
CT252 t252 0 0.1f
M681 t252 nw28 vdd vdd pch w=2u l=180n
M682 t252 nw80 vdd vdd pch w=2u l=180n
CT253 t253 0 0.1f
M683 t252 nw28 t253 0 nch w=1u l=180n
M684 t253 nw80 0 0 nch w=1u l=180n
M685 nw90 t252 vdd vdd pch w=2u l=180n
M686 nw90 t252 0 0 nch w=1u l=180n
Cnw90 nw90 0 2f
CT254 t254 0 0.1f
M687 t254 nw29 0 0 nch w=1u l=180n
M688 t254 nw82 0 0 nch w=1u l=180n
CT255 t255 0 0.1f
M689 t255 nw29 vdd vdd pch w=2u l=180n
M690 t254 nw82 t255 vdd pch w=2u l=180n
M691 nw91 t254 vdd vdd pch w=2u l=180n
M692 nw91 t254 0 0 nch w=1u l=180n
Cnw91 nw91 0 2f
CT256 t256 0 0.1f
CT257 t257 0 0.1f
CT258 t258 0 0.1f
M693 t256 nw30 vdd vdd pch w=2u l=180n
M694 t256 nw84 vdd vdd pch w=2u l=180n
CT259 t259 0 0.1f
M695 t256 nw30 t259 0 nch w=1u l=180n
M696 t259 nw84 0 0 nch w=1u l=180n
M697 t257 nw30 vdd vdd pch w=2u l=180n
M698 t257 t256 vdd vdd pch w=2u l=180n
CT260 t260 0 0.1f
M699 t257 nw30 t260 0 nch w=1u l=180n
M700 t260 t256 0 0 nch w=1u l=180n
M701 t258 nw84 vdd vdd pch w=2u l=180n
M702 t258 t256 vdd vdd pch w=2u l=180n
CT261 t261 0 0.1f
M703 t258 nw84 t261 0 nch w=1u l=180n
M704 t261 t256 0 0 nch w=1u l=180n
M705 nw92 t257 vdd vdd pch w=2u l=180n
M706 nw92 t258 vdd vdd pch w=2u l=180n
CT262 t262 0 0.1f
M707 nw92 t257 t262 0 nch w=1u l=180n
M708 t262 t258 0 0 nch w=1u l=180n
Cnw92 nw92 0 2f
M709 nw93 nw31 vdd vdd pch w=2u l=180n
M710 nw93 nw86 vdd vdd pch w=2u l=180n
CT263 t263 0 0.1f
M711 nw93 nw31 t263 0 nch w=1u l=180n
M712 t263 nw86 0 0 nch w=1u l=180n
Cnw93 nw93 0 2f
M713 nw94 nw32 0 0 nch w=1u l=180n
M714 nw94 nw88 0 0 nch w=1u l=180n
CT264 t264 0 0.1f
M715 t264 nw32 vdd vdd pch w=2u l=180n
M716 nw94 nw88 t264 vdd pch w=2u l=180n
Cnw94 nw94 0 2f
CT265 t265 0 0.1f
M717 t265 nw33 vdd vdd pch w=2u l=180n
M718 t265 nw90 vdd vdd pch w=2u l=180n
CT266 t266 0 0.1f
M719 t265 nw33 t266 0 nch w=1u l=180n
M720 t266 nw90 0 0 nch w=1u l=180n
M721 nw95 t265 vdd vdd pch w=2u l=180n
M722 nw95 t265 0 0 nch w=1u l=180n
Cnw95 nw95 0 2f
CT267 t267 0 0.1f
M723 t267 nw34 0 0 nch w=1u l=180n
M724 t267 nw92 0 0 nch w=1u l=180n
CT268 t268 0 0.1f
M725 t268 nw34 vdd vdd pch w=2u l=180n
M726 t267 nw92 t268 vdd pch w=2u l=180n
M727 nw96 t267 vdd vdd pch w=2u l=180n
M728 nw96 t267 0 0 nch w=1u l=180n
Cnw96 nw96 0 2f
CT269 t269 0 0.1f
CT270 t270 0 0.1f
CT271 t271 0 0.1f
M729 t269 nw35 vdd vdd pch w=2u l=180n
M730 t269 nw94 vdd vdd pch w=2u l=180n
CT272 t272 0 0.1f
M731 t269 nw35 t272 0 nch w=1u l=180n
M732 t272 nw94 0 0 nch w=1u l=180n
M733 t270 nw35 vdd vdd pch w=2u l=180n
M734 t270 t269 vdd vdd pch w=2u l=180n
CT273 t273 0 0.1f
M735 t270 nw35 t273 0 nch w=1u l=180n
M736 t273 t269 0 0 nch w=1u l=180n
M737 t271 nw94 vdd vdd pch w=2u l=180n
M738 t271 t269 vdd vdd pch w=2u l=180n
CT274 t274 0 0.1f
M739 t271 nw94 t274 0 nch w=1u l=180n
M740 t274 t269 0 0 nch w=1u l=180n
M741 nw97 t270 vdd vdd pch w=2u l=180n
M742 nw97 t271 vdd vdd pch w=2u l=180n
CT275 t275 0 0.1f
M743 nw97 t270 t275 0 nch w=1u l=180n
M744 t275 t271 0 0 nch w=1u l=180n
Cnw97 nw97 0 2f
M745 nw98 nw36 vdd vdd pch w=2u l=180n
M746 nw98 nw96 vdd vdd pch w=2u l=180n
CT276 t276 0 0.1f
M747 nw98 nw36 t276 0 nch w=1u l=180n
M748 t276 nw96 0 0 nch w=1u l=180n
Cnw98 nw98 0 2f
M749 nw99 nw37 0 0 nch w=1u l=180n
M750 nw99 nw98 0 0 nch w=1u l=180n
CT277 t277 0 0.1f
M751 t277 nw37 vdd vdd pch w=2u l=180n
M752 nw99 nw98 t277 vdd pch w=2u l=180n
Cnw99 nw99 0 2f
CT278 t278 0 0.1f
M753 t278 nw38 vdd vdd pch w=2u l=180n
M754 t278 nq0 vdd vdd pch w=2u l=180n
CT279 t279 0 0.1f
M755 t278 nw38 t279 0 nch w=1u l=180n
M756 t279 nq0 0 0 nch w=1u l=180n
M757 nw100 t278 vdd vdd pch w=2u l=180n
M758 nw100 t278 0 0 nch w=1u l=180n
Cnw100 nw100 0 2f
CT280 t280 0 0.1f
M759 t280 nw39 0 0 nch w=1u l=180n
M760 t280 nq1 0 0 nch w=1u l=180n
CT281 t281 0 0.1f
M761 t281 nw39 vdd vdd pch w=2u l=180n
M762 t280 nq1 t281 vdd pch w=2u l=180n
M763 nw101 t280 vdd vdd pch w=2u l=180n
M764 nw101 t280 0 0 nch w=1u l=180n
Cnw101 nw101 0 2f
CT282 t282 0 0.1f
CT283 t283 0 0.1f
CT284 t284 0 0.1f
M765 t282 nw40 vdd vdd pch w=2u l=180n
M766 t282 nq2 vdd vdd pch w=2u l=180n
CT285 t285 0 0.1f
M767 t282 nw40 t285 0 nch w=1u l=180n
M768 t285 nq2 0 0 nch w=1u l=180n
M769 t283 nw40 vdd vdd pch w=2u l=180n
M770 t283 t282 vdd vdd pch w=2u l=180n
CT286 t286 0 0.1f
M771 t283 nw40 t286 0 nch w=1u l=180n
M772 t286 t282 0 0 nch w=1u l=180n
M773 t284 nq2 vdd vdd pch w=2u l=180n
M774 t284 t282 vdd vdd pch w=2u l=180n
CT287 t287 0 0.1f
M775 t284 nq2 t287 0 nch w=1u l=180n
M776 t287 t282 0 0 nch w=1u l=180n
M777 nw102 t283 vdd vdd pch w=2u l=180n
M778 nw102 t284 vdd vdd pch w=2u l=180n
CT288 t288 0 0.1f
M779 nw102 t283 t288 0 nch w=1u l=180n
M780 t288 t284 0 0 nch w=1u l=180n
Cnw102 nw102 0 2f
M781 nw103 nw41 vdd vdd pch w=2u l=180n
M782 nw103 nq3 vdd vdd pch w=2u l=180n
CT289 t289 0 0.1f
M783 nw103 nw41 t289 0 nch w=1u l=180n
M784 t289 nq3 0 0 nch w=1u l=180n
Cnw103 nw103 0 2f
M785 nw104 nw42 0 0 nch w=1u l=180n
M786 nw104 nq4 0 0 nch w=1u l=180n
CT290 t290 0 0.1f
M787 t290 nw42 vdd vdd pch w=2u l=180n
M788 nw104 nq4 t290 vdd pch w=2u l=180n
Cnw104 nw104 0 2f
CT291 t291 0 0.1f
M789 t291 nw43 vdd vdd pch w=2u l=180n
M790 t291 nq5 vdd vdd pch w=2u l=180n
CT292 t292 0 0.1f
M791 t291 nw43 t292 0 nch w=1u l=180n
M792 t292 nq5 0 0 nch w=1u l=180n
M793 nw105 t291 vdd vdd pch w=2u l=180n
M794 nw105 t291 0 0 nch w=1u l=180n
Cnw105 nw105 0 2f
CT293 t293 0 0.1f
M795 t293 nw44 0 0 nch w=1u l=180n
M796 t293 ni0 0 0 nch w=1u l=180n
CT294 t294 0 0.1f
M797 t294 nw44 vdd vdd pch w=2u l=180n
M798 t293 ni0 t294 vdd pch w=2u l=180n
M799 nw106 t293 vdd vdd pch w=2u l=180n
M800 nw106 t293 0 0 nch w=1u l=180n
Cnw106 nw106 0 2f
CT295 t295 0 0.1f
CT296 t296 0 0.1f
CT297 t297 0 0.1f
M801 t295 nw45 vdd vdd pch w=2u l=180n
M802 t295 ni1 vdd vdd pch w=2u l=180n
CT298 t298 0 0.1f
M803 t295 nw45 t298 0 nch w=1u l=180n
M804 t298 ni1 0 0 nch w=1u l=180n
M805 t296 nw45 vdd vdd pch w=2u l=180n
M806 t296 t295 vdd vdd pch w=2u l=180n
CT299 t299 0 0.1f
M807 t296 nw45 t299 0 nch w=1u l=180n
M808 t299 t295 0 0 nch w=1u l=180n
M809 t297 ni1 vdd vdd pch w=2u l=180n
M810 t297 t295 vdd vdd pch w=2u l=180n
CT300 t300 0 0.1f
M811 t297 ni1 t300 0 nch w=1u l=180n
M812 t300 t295 0 0 nch w=1u l=180n
M813 nw107 t296 vdd vdd pch w=2u l=180n
M814 nw107 t297 vdd vdd pch w=2u l=180n
CT301 t301 0 0.1f
M815 nw107 t296 t301 0 nch w=1u l=180n
M816 t301 t297 0 0 nch w=1u l=180n
Cnw107 nw107 0 2f
M817 nw108 nw46 vdd vdd pch w=2u l=180n
M818 nw108 ni2 vdd vdd pch w=2u l=180n
CT302 t302 0 0.1f
M819 nw108 nw46 t302 0 nch w=1u l=180n
M820 t302 ni2 0 0 nch w=1u l=180n
Cnw108 nw108 0 2f
M821 nw109 nw47 0 0 nch w=1u l=180n
M822 nw109 nw13 0 0 nch w=1u l=180n
CT303 t303 0 0.1f
M823 t303 nw47 vdd vdd pch w=2u l=180n
M824 nw109 nw13 t303 vdd pch w=2u l=180n
Cnw109 nw109 0 2f
CT304 t304 0 0.1f
M825 t304 nw48 vdd vdd pch w=2u l=180n
M826 t304 nw14 vdd vdd pch w=2u l=180n
CT305 t305 0 0.1f
M827 t304 nw48 t305 0 nch w=1u l=180n
M828 t305 nw14 0 0 nch w=1u l=180n
M829 nw110 t304 vdd vdd pch w=2u l=180n
M830 nw110 t304 0 0 nch w=1u l=180n
Cnw110 nw110 0 2f
CT306 t306 0 0.1f
M831 t306 nw49 0 0 nch w=1u l=180n
M832 t306 nw15 0 0 nch w=1u l=180n
CT307 t307 0 0.1f
M833 t307 nw49 vdd vdd pch w=2u l=180n
M834 t306 nw15 t307 vdd pch w=2u l=180n
M835 nw111 t306 vdd vdd pch w=2u l=180n
M836 nw111 t306 0 0 nch w=1u l=180n
Cnw111 nw111 0 2f
CT308 t308 0 0.1f
CT309 t309 0 0.1f
CT310 t310 0 0.1f
M837 t308 nw50 vdd vdd pch w=2u l=180n
M838 t308 nw16 vdd vdd pch w=2u l=180n
CT311 t311 0 0.1f
M839 t308 nw50 t311 0 nch w=1u l=180n
M840 t311 nw16 0 0 nch w=1u l=180n
M841 t309 nw50 vdd vdd pch w=2u l=180n
M842 t309 t308 vdd vdd pch w=2u l=180n
CT312 t312 0 0.1f
M843 t309 nw50 t312 0 nch w=1u l=180n
M844 t312 t308 0 0 nch w=1u l=180n
M845 t310 nw16 vdd vdd pch w=2u l=180n
M846 t310 t308 vdd vdd pch w=2u l=180n
CT313 t313 0 0.1f
M847 t310 nw16 t313 0 nch w=1u l=180n
M848 t313 t308 0 0 nch w=1u l=180n
M849 nw112 t309 vdd vdd pch w=2u l=180n
M850 nw112 t310 vdd vdd pch w=2u l=180n
CT314 t314 0 0.1f
M851 nw112 t309 t314 0 nch w=1u l=180n
M852 t314 t310 0 0 nch w=1u l=180n
Cnw112 nw112 0 2f
M853 nw113 nw51 vdd vdd pch w=2u l=180n
M854 nw113 nw17 vdd vdd pch w=2u l=180n
CT315 t315 0 0.1f
M855 nw113 nw51 t315 0 nch w=1u l=180n
M856 t315 nw17 0 0 nch w=1u l=180n
Cnw113 nw113 0 2f
M857 nw114 nw52 0 0 nch w=1u l=180n
M858 nw114 nw18 0 0 nch w=1u l=180n
CT316 t316 0 0.1f
M859 t316 nw52 vdd vdd pch w=2u l=180n
M860 nw114 nw18 t316 vdd pch w=2u l=180n
Cnw114 nw114 0 2f
CT317 t317 0 0.1f
M861 t317 nw53 vdd vdd pch w=2u l=180n
M862 t317 nw19 vdd vdd pch w=2u l=180n
CT318 t318 0 0.1f
M863 t317 nw53 t318 0 nch w=1u l=180n
M864 t318 nw19 0 0 nch w=1u l=180n
M865 nw115 t317 vdd vdd pch w=2u l=180n
M866 nw115 t317 0 0 nch w=1u l=180n
Cnw115 nw115 0 2f
CT319 t319 0 0.1f
M867 t319 nw54 0 0 nch w=1u l=180n
M868 t319 nw20 0 0 nch w=1u l=180n
CT320 t320 0 0.1f
M869 t320 nw54 vdd vdd pch w=2u l=180n
M870 t319 nw20 t320 vdd pch w=2u l=180n
M871 nw116 t319 vdd vdd pch w=2u l=180n
M872 nw116 t319 0 0 nch w=1u l=180n
Cnw116 nw116 0 2f
CT321 t321 0 0.1f
CT322 t322 0 0.1f
CT323 t323 0 0.1f
M873 t321 nw55 vdd vdd pch w=2u l=180n
M874 t321 nw21 vdd vdd pch w=2u l=180n
CT324 t324 0 0.1f
M875 t321 nw55 t324 0 nch w=1u l=180n
M876 t324 nw21 0 0 nch w=1u l=180n
M877 t322 nw55 vdd vdd pch w=2u l=180n
M878 t322 t321 vdd vdd pch w=2u l=180n
CT325 t325 0 0.1f
M879 t322 nw55 t325 0 nch w=1u l=180n
M880 t325 t321 0 0 nch w=1u l=180n
M881 t323 nw21 vdd vdd pch w=2u l=180n
M882 t323 t321 vdd vdd pch w=2u l=180n
CT326 t326 0 0.1f
M883 t323 nw21 t326 0 nch w=1u l=180n
M884 t326 t321 0 0 nch w=1u l=180n
M885 nw117 t322 vdd vdd pch w=2u l=180n
M886 nw117 t323 vdd vdd pch w=2u l=180n
CT327 t327 0 0.1f
M887 nw117 t322 t327 0 nch w=1u l=180n
M888 t327 t323 0 0 nch w=1u l=180n
Cnw117 nw117 0 2f
M889 nw118 nw56 vdd vdd pch w=2u l=180n
M890 nw118 nw22 vdd vdd pch w=2u l=180n
CT328 t328 0 0.1f
M891 nw118 nw56 t328 0 nch w=1u l=180n
M892 t328 nw22 0 0 nch w=1u l=180n
Cnw118 nw118 0 2f
M893 nw119 nw57 0 0 nch w=1u l=180n
M894 nw119 nw23 0 0 nch w=1u l=180n
CT329 t329 0 0.1f
M895 t329 nw57 vdd vdd pch w=2u l=180n
M896 nw119 nw23 t329 vdd pch w=2u l=180n
Cnw119 nw119 0 2f
CT330 t330 0 0.1f
M897 t330 nw58 vdd vdd pch w=2u l=180n
M898 t330 nw24 vdd vdd pch w=2u l=180n
CT331 t331 0 0.1f
M899 t330 nw58 t331 0 nch w=1u l=180n
M900 t331 nw24 0 0 nch w=1u l=180n
M901 nw120 t330 vdd vdd pch w=2u l=180n
M902 nw120 t330 0 0 nch w=1u l=180n
Cnw120 nw120 0 2f
CT332 t332 0 0.1f
M903 t332 nw59 0 0 nch w=1u l=180n
M904 t332 nw25 0 0 nch w=1u l=180n
CT333 t333 0 0.1f
M905 t333 nw59 vdd vdd pch w=2u l=180n
M906 t332 nw25 t333 vdd pch w=2u l=180n
M907 nw121 t332 vdd vdd pch w=2u l=180n
M908 nw121 t332 0 0 nch w=1u l=180n
Cnw121 nw121 0 2f
CT334 t334 0 0.1f
CT335 t335 0 0.1f
CT336 t336 0 0.1f
M909 t334 nw60 vdd vdd pch w=2u l=180n
M910 t334 nw26 vdd vdd pch w=2u l=180n
CT337 t337 0 0.1f
M911 t334 nw60 t337 0 nch w=1u l=180n
M912 t337 nw26 0 0 nch w=1u l=180n
M913 t335 nw60 vdd vdd pch w=2u l=180n
M914 t335 t334 vdd vdd pch w=2u l=180n
CT338 t338 0 0.1f
M915 t335 nw60 t338 0 nch w=1u l=180n
M916 t338 t334 0 0 nch w=1u l=180n
M917 t336 nw26 vdd vdd pch w=2u l=180n
M918 t336 t334 vdd vdd pch w=2u l=180n
CT339 t339 0 0.1f
M919 t336 nw26 t339 0 nch w=1u l=180n
M920 t339 t334 0 0 nch w=1u l=180n
M921 nw122 t335 vdd vdd pch w=2u l=180n
M922 nw122 t336 vdd vdd pch w=2u l=180n
CT340 t340 0 0.1f
M923 nw122 t335 t340 0 nch w=1u l=180n
M924 t340 t336 0 0 nch w=1u l=180n
Cnw122 nw122 0 2f
M925 nw123 nw61 vdd vdd pch w=2u l=180n
M926 nw123 nw27 vdd vdd pch w=2u l=180n
CT341 t341 0 0.1f
M927 nw123 nw61 t341 0 nch w=1u l=180n
M928 t341 nw27 0 0 nch w=1u l=180n
Cnw123 nw123 0 2f
M929 nw124 nw62 0 0 nch w=1u l=180n
M930 nw124 nw28 0 0 nch w=1u l=180n
CT342 t342 0 0.1f
M931 t342 nw62 vdd vdd pch w=2u l=180n
M932 nw124 nw28 t342 vdd pch w=2u l=180n
Cnw124 nw124 0 2f
CT343 t343 0 0.1f
M933 t343 nw63 vdd vdd pch w=2u l=180n
M934 t343 nw29 vdd vdd pch w=2u l=180n
CT344 t344 0 0.1f
M935 t343 nw63 t344 0 nch w=1u l=180n
M936 t344 nw29 0 0 nch w=1u l=180n
M937 nw125 t343 vdd vdd pch w=2u l=180n
M938 nw125 t343 0 0 nch w=1u l=180n
Cnw125 nw125 0 2f
CT345 t345 0 0.1f
M939 t345 nw64 0 0 nch w=1u l=180n
M940 t345 nw30 0 0 nch w=1u l=180n
CT346 t346 0 0.1f
M941 t346 nw64 vdd vdd pch w=2u l=180n
M942 t345 nw30 t346 vdd pch w=2u l=180n
M943 nw126 t345 vdd vdd pch w=2u l=180n
M944 nw126 t345 0 0 nch w=1u l=180n
Cnw126 nw126 0 2f
CT347 t347 0 0.1f
CT348 t348 0 0.1f
CT349 t349 0 0.1f
M945 t347 nw65 vdd vdd pch w=2u l=180n
M946 t347 nw31 vdd vdd pch w=2u l=180n
CT350 t350 0 0.1f
M947 t347 nw65 t350 0 nch w=1u l=180n
M948 t350 nw31 0 0 nch w=1u l=180n
M949 t348 nw65 vdd vdd pch w=2u l=180n
M950 t348 t347 vdd vdd pch w=2u l=180n
CT351 t351 0 0.1f
M951 t348 nw65 t351 0 nch w=1u l=180n
M952 t351 t347 0 0 nch w=1u l=180n
M953 t349 nw31 vdd vdd pch w=2u l=180n
M954 t349 t347 vdd vdd pch w=2u l=180n
CT352 t352 0 0.1f
M955 t349 nw31 t352 0 nch w=1u l=180n
M956 t352 t347 0 0 nch w=1u l=180n
M957 nw127 t348 vdd vdd pch w=2u l=180n
M958 nw127 t349 vdd vdd pch w=2u l=180n
CT353 t353 0 0.1f
M959 nw127 t348 t353 0 nch w=1u l=180n
M960 t353 t349 0 0 nch w=1u l=180n
Cnw127 nw127 0 2f
M961 nw128 nw66 vdd vdd pch w=2u l=180n
M962 nw128 nw32 vdd vdd pch w=2u l=180n
CT354 t354 0 0.1f
M963 nw128 nw66 t354 0 nch w=1u l=180n
M964 t354 nw32 0 0 nch w=1u l=180n
Cnw128 nw128 0 2f
M965 nw129 nw67 0 0 nch w=1u l=180n
M966 nw129 nw33 0 0 nch w=1u l=180n
CT355 t355 0 0.1f
M967 t355 nw67 vdd vdd pch w=2u l=180n
M968 nw129 nw33 t355 vdd pch w=2u l=180n
Cnw129 nw129 0 2f
CT356 t356 0 0.1f
M969 t356 nw68 vdd vdd pch w=2u l=180n
M970 t356 nw34 vdd vdd pch w=2u l=180n
CT357 t357 0 0.1f
M971 t356 nw68 t357 0 nch w=1u l=180n
M972 t357 nw34 0 0 nch w=1u l=180n
M973 nw130 t356 vdd vdd pch w=2u l=180n
M974 nw130 t356 0 0 nch w=1u l=180n
Cnw130 nw130 0 2f
CT358 t358 0 0.1f
M975 t358 nw69 0 0 nch w=1u l=180n
M976 t358 nw35 0 0 nch w=1u l=180n
CT359 t359 0 0.1f
M977 t359 nw69 vdd vdd pch w=2u l=180n
M978 t358 nw35 t359 vdd pch w=2u l=180n
M979 nw131 t358 vdd vdd pch w=2u l=180n
M980 nw131 t358 0 0 nch w=1u l=180n
Cnw131 nw131 0 2f
CT360 t360 0 0.1f
CT361 t361 0 0.1f
CT362 t362 0 0.1f
M981 t360 nw70 vdd vdd pch w=2u l=180n
M982 t360 nw36 vdd vdd pch w=2u l=180n
CT363 t363 0 0.1f
M983 t360 nw70 t363 0 nch w=1u l=180n
M984 t363 nw36 0 0 nch w=1u l=180n
M985 t361 nw70 vdd vdd pch w=2u l=180n
M986 t361 t360 vdd vdd pch w=2u l=180n
CT364 t364 0 0.1f
M987 t361 nw70 t364 0 nch w=1u l=180n
M988 t364 t360 0 0 nch w=1u l=180n
M989 t362 nw36 vdd vdd pch w=2u l=180n
M990 t362 t360 vdd vdd pch w=2u l=180n
CT365 t365 0 0.1f
M991 t362 nw36 t365 0 nch w=1u l=180n
M992 t365 t360 0 0 nch w=1u l=180n
M993 nw132 t361 vdd vdd pch w=2u l=180n
M994 nw132 t362 vdd vdd pch w=2u l=180n
CT366 t366 0 0.1f
M995 nw132 t361 t366 0 nch w=1u l=180n
M996 t366 t362 0 0 nch w=1u l=180n
Cnw132 nw132 0 2f
M997 nw133 nw71 vdd vdd pch w=2u l=180n
M998 nw133 nw37 vdd vdd pch w=2u l=180n
CT367 t367 0 0.1f
M999 nw133 nw71 t367 0 nch w=1u l=180n
M1000 t367 nw37 0 0 nch w=1u l=180n
Cnw133 nw133 0 2f
M1001 nw134 nw72 0 0 nch w=1u l=180n
M1002 nw134 nw38 0 0 nch w=1u l=180n
CT368 t368 0 0.1f
M1003 t368 nw72 vdd vdd pch w=2u l=180n
M1004 nw134 nw38 t368 vdd pch w=2u l=180n
Cnw134 nw134 0 2f
CT369 t369 0 0.1f
M1005 t369 nw73 vdd vdd pch w=2u l=180n
M1006 t369 nw39 vdd vdd pch w=2u l=180n
CT370 t370 0 0.1f
M1007 t369 nw73 t370 0 nch w=1u l=180n
M1008 t370 nw39 0 0 nch w=1u l=180n
M1009 nw135 t369 vdd vdd pch w=2u l=180n
M1010 nw135 t369 0 0 nch w=1u l=180n
Cnw135 nw135 0 2f
CT371 t371 0 0.1f
M1011 t371 nw74 0 0 nch w=1u l=180n
M1012 t371 nw40 0 0 nch w=1u l=180n
CT372 t372 0 0.1f
M1013 t372 nw74 vdd vdd pch w=2u l=180n
M1014 t371 nw40 t372 vdd pch w=2u l=180n
M1015 nw136 t371 vdd vdd pch w=2u l=180n
M1016 nw136 t371 0 0 nch w=1u l=180n
Cnw136 nw136 0 2f
CT373 t373 0 0.1f
CT374 t374 0 0.1f
CT375 t375 0 0.1f
M1017 t373 nw75 vdd vdd pch w=2u l=180n
M1018 t373 nw41 vdd vdd pch w=2u l=180n
CT376 t376 0 0.1f
M1019 t373 nw75 t376 0 nch w=1u l=180n
M1020 t376 nw41 0 0 nch w=1u l=180n
M1021 t374 nw75 vdd vdd pch w=2u l=180n
M1022 t374 t373 vdd vdd pch w=2u l=180n
CT377 t377 0 0.1f
M1023 t374 nw75 t377 0 nch w=1u l=180n
M1024 t377 t373 0 0 nch w=1u l=180n
M1025 t375 nw41 vdd vdd pch w=2u l=180n
M1026 t375 t373 vdd vdd pch w=2u l=180n
CT378 t378 0 0.1f
M1027 t375 nw41 t378 0 nch w=1u l=180n
M1028 t378 t373 0 0 nch w=1u l=180n
M1029 nw137 t374 vdd vdd pch w=2u l=180n
M1030 nw137 t375 vdd vdd pch w=2u l=180n
CT379 t379 0 0.1f
M1031 nw137 t374 t379 0 nch w=1u l=180n
M1032 t379 t375 0 0 nch w=1u l=180n
Cnw137 nw137 0 2f
M1033 nw138 nw76 vdd vdd pch w=2u l=180n
M1034 nw138 nw42 vdd vdd pch w=2u l=180n
CT380 t380 0 0.1f
M1035 nw138 nw76 t380 0 nch w=1u l=180n
M1036 t380 nw42 0 0 nch w=1u l=180n
Cnw138 nw138 0 2f
M1037 nw139 nw77 0 0 nch w=1u l=180n
M1038 nw139 nw43 0 0 nch w=1u l=180n
CT381 t381 0 0.1f
M1039 t381 nw77 vdd vdd pch w=2u l=180n
M1040 nw139 nw43 t381 vdd pch w=2u l=180n
Cnw139 nw139 0 2f
CT382 t382 0 0.1f
M1041 t382 nw78 vdd vdd pch w=2u l=180n
M1042 t382 nw44 vdd vdd pch w=2u l=180n
CT383 t383 0 0.1f
M1043 t382 nw78 t383 0 nch w=1u l=180n
M1044 t383 nw44 0 0 nch w=1u l=180n
M1045 nw140 t382 vdd vdd pch w=2u l=180n
M1046 nw140 t382 0 0 nch w=1u l=180n
Cnw140 nw140 0 2f
CT384 t384 0 0.1f
M1047 t384 nw79 0 0 nch w=1u l=180n
M1048 t384 nw45 0 0 nch w=1u l=180n
CT385 t385 0 0.1f
M1049 t385 nw79 vdd vdd pch w=2u l=180n
M1050 t384 nw45 t385 vdd pch w=2u l=180n
M1051 nw141 t384 vdd vdd pch w=2u l=180n
M1052 nw141 t384 0 0 nch w=1u l=180n
Cnw141 nw141 0 2f
CT386 t386 0 0.1f
CT387 t387 0 0.1f
CT388 t388 0 0.1f
M1053 t386 nw80 vdd vdd pch w=2u l=180n
M1054 t386 nw46 vdd vdd pch w=2u l=180n
CT389 t389 0 0.1f
M1055 t386 nw80 t389 0 nch w=1u l=180n
M1056 t389 nw46 0 0 nch w=1u l=180n
M1057 t387 nw80 vdd vdd pch w=2u l=180n
M1058 t387 t386 vdd vdd pch w=2u l=180n
CT390 t390 0 0.1f
M1059 t387 nw80 t390 0 nch w=1u l=180n
M1060 t390 t386 0 0 nch w=1u l=180n
M1061 t388 nw46 vdd vdd pch w=2u l=180n
M1062 t388 t386 vdd vdd pch w=2u l=180n
CT391 t391 0 0.1f
M1063 t388 nw46 t391 0 nch w=1u l=180n
M1064 t391 t386 0 0 nch w=1u l=180n
M1065 nw142 t387 vdd vdd pch w=2u l=180n
M1066 nw142 t388 vdd vdd pch w=2u l=180n
CT392 t392 0 0.1f
M1067 nw142 t387 t392 0 nch w=1u l=180n
M1068 t392 t388 0 0 nch w=1u l=180n
Cnw142 nw142 0 2f
M1069 nw143 nw81 vdd vdd pch w=2u l=180n
M1070 nw143 nw47 vdd vdd pch w=2u l=180n
CT393 t393 0 0.1f
M1071 nw143 nw81 t393 0 nch w=1u l=180n
M1072 t393 nw47 0 0 nch w=1u l=180n
Cnw143 nw143 0 2f
M1073 nw144 nw82 0 0 nch w=1u l=180n
M1074 nw144 nw48 0 0 nch w=1u l=180n
CT394 t394 0 0.1f
M1075 t394 nw82 vdd vdd pch w=2u l=180n
M1076 nw144 nw48 t394 vdd pch w=2u l=180n
Cnw144 nw144 0 2f
CT395 t395 0 0.1f
M1077 t395 nw83 vdd vdd pch w=2u l=180n
M1078 t395 nw49 vdd vdd pch w=2u l=180n
CT396 t396 0 0.1f
M1079 t395 nw83 t396 0 nch w=1u l=180n
M1080 t396 nw49 0 0 nch w=1u l=180n
M1081 nw145 t395 vdd vdd pch w=2u l=180n
M1082 nw145 t395 0 0 nch w=1u l=180n
Cnw145 nw145 0 2f
CT397 t397 0 0.1f
M1083 t397 nw84 0 0 nch w=1u l=180n
M1084 t397 nw50 0 0 nch w=1u l=180n
CT398 t398 0 0.1f
M1085 t398 nw84 vdd vdd pch w=2u l=180n
M1086 t397 nw50 t398 vdd pch w=2u l=180n
M1087 nw146 t397 vdd vdd pch w=2u l=180n
M1088 nw146 t397 0 0 nch w=1u l=180n
Cnw146 nw146 0 2f
CT399 t399 0 0.1f
CT400 t400 0 0.1f
CT401 t401 0 0.1f
M1089 t399 nw85 vdd vdd pch w=2u l=180n
M1090 t399 nw51 vdd vdd pch w=2u l=180n
CT402 t402 0 0.1f
M1091 t399 nw85 t402 0 nch w=1u l=180n
M1092 t402 nw51 0 0 nch w=1u l=180n
M1093 t400 nw85 vdd vdd pch w=2u l=180n
M1094 t400 t399 vdd vdd pch w=2u l=180n
CT403 t403 0 0.1f
M1095 t400 nw85 t403 0 nch w=1u l=180n
M1096 t403 t399 0 0 nch w=1u l=180n
M1097 t401 nw51 vdd vdd pch w=2u l=180n
M1098 t401 t399 vdd vdd pch w=2u l=180n
CT404 t404 0 0.1f
M1099 t401 nw51 t404 0 nch w=1u l=180n
M1100 t404 t399 0 0 nch w=1u l=180n
M1101 nw147 t400 vdd vdd pch w=2u l=180n
M1102 nw147 t401 vdd vdd pch w=2u l=180n
CT405 t405 0 0.1f
M1103 nw147 t400 t405 0 nch w=1u l=180n
M1104 t405 t401 0 0 nch w=1u l=180n
Cnw147 nw147 0 2f
M1105 nw148 nw86 vdd vdd pch w=2u l=180n
M1106 nw148 nw52 vdd vdd pch w=2u l=180n
CT406 t406 0 0.1f
M1107 nw148 nw86 t406 0 nch w=1u l=180n
M1108 t406 nw52 0 0 nch w=1u l=180n
Cnw148 nw148 0 2f
M1109 nw149 nw87 0 0 nch w=1u l=180n
M1110 nw149 nw53 0 0 nch w=1u l=180n
CT407 t407 0 0.1f
M1111 t407 nw87 vdd vdd pch w=2u l=180n
M1112 nw149 nw53 t407 vdd pch w=2u l=180n
Cnw149 nw149 0 2f
CT408 t408 0 0.1f
M1113 t408 nw88 vdd vdd pch w=2u l=180n
M1114 t408 nw54 vdd vdd pch w=2u l=180n
CT409 t409 0 0.1f
M1115 t408 nw88 t409 0 nch w=1u l=180n
M1116 t409 nw54 0 0 nch w=1u l=180n
M1117 nw150 t408 vdd vdd pch w=2u l=180n
M1118 nw150 t408 0 0 nch w=1u l=180n
Cnw150 nw150 0 2f
CT410 t410 0 0.1f
M1119 t410 nw89 0 0 nch w=1u l=180n
M1120 t410 nw55 0 0 nch w=1u l=180n
CT411 t411 0 0.1f
M1121 t411 nw89 vdd vdd pch w=2u l=180n
M1122 t410 nw55 t411 vdd pch w=2u l=180n
M1123 nw151 t410 vdd vdd pch w=2u l=180n
M1124 nw151 t410 0 0 nch w=1u l=180n
Cnw151 nw151 0 2f
CT412 t412 0 0.1f
CT413 t413 0 0.1f
CT414 t414 0 0.1f
M1125 t412 nw90 vdd vdd pch w=2u l=180n
M1126 t412 nw56 vdd vdd pch w=2u l=180n
CT415 t415 0 0.1f
M1127 t412 nw90 t415 0 nch w=1u l=180n
M1128 t415 nw56 0 0 nch w=1u l=180n
M1129 t413 nw90 vdd vdd pch w=2u l=180n
M1130 t413 t412 vdd vdd pch w=2u l=180n
CT416 t416 0 0.1f
M1131 t413 nw90 t416 0 nch w=1u l=180n
M1132 t416 t412 0 0 nch w=1u l=180n
M1133 t414 nw56 vdd vdd pch w=2u l=180n
M1134 t414 t412 vdd vdd pch w=2u l=180n
CT417 t417 0 0.1f
M1135 t414 nw56 t417 0 nch w=1u l=180n
M1136 t417 t412 0 0 nch w=1u l=180n
M1137 nw152 t413 vdd vdd pch w=2u l=180n
M1138 nw152 t414 vdd vdd pch w=2u l=180n
CT418 t418 0 0.1f
M1139 nw152 t413 t418 0 nch w=1u l=180n
M1140 t418 t414 0 0 nch w=1u l=180n
Cnw152 nw152 0 2f
M1141 nw153 nw91 vdd vdd pch w=2u l=180n
M1142 nw153 nw57 vdd vdd pch w=2u l=180n
CT419 t419 0 0.1f
M1143 nw153 nw91 t419 0 nch w=1u l=180n
M1144 t419 nw57 0 0 nch w=1u l=180n
Cnw153 nw153 0 2f
M1145 nw154 nw92 0 0 nch w=1u l=180n
M1146 nw154 nw58 0 0 nch w=1u l=180n
CT420 t420 0 0.1f
M1147 t420 nw92 vdd vdd pch w=2u l=180n
M1148 nw154 nw58 t420 vdd pch w=2u l=180n
Cnw154 nw154 0 2f
CT421 t421 0 0.1f
M1149 t421 nw93 vdd vdd pch w=2u l=180n
M1150 t421 nw59 vdd vdd pch w=2u l=180n
CT422 t422 0 0.1f
M1151 t421 nw93 t422 0 nch w=1u l=180n
M1152 t422 nw59 0 0 nch w=1u l=180n
M1153 nw155 t421 vdd vdd pch w=2u l=180n
M1154 nw155 t421 0 0 nch w=1u l=180n
Cnw155 nw155 0 2f
CT423 t423 0 0.1f
M1155 t423 nw94 0 0 nch w=1u l=180n
M1156 t423 nw60 0 0 nch w=1u l=180n
CT424 t424 0 0.1f
M1157 t424 nw94 vdd vdd pch w=2u l=180n
M1158 t423 nw60 t424 vdd pch w=2u l=180n
M1159 nw156 t423 vdd vdd pch w=2u l=180n
M1160 nw156 t423 0 0 nch w=1u l=180n
Cnw156 nw156 0 2f
CT425 t425 0 0.1f
CT426 t426 0 0.1f
CT427 t427 0 0.1f
M1161 t425 nw95 vdd vdd pch w=2u l=180n
M1162 t425 nw61 vdd vdd pch w=2u l=180n
CT428 t428 0 0.1f
M1163 t425 nw95 t428 0 nch w=1u l=180n
M1164 t428 nw61 0 0 nch w=1u l=180n
M1165 t426 nw95 vdd vdd pch w=2u l=180n
M1166 t426 t425 vdd vdd pch w=2u l=180n
CT429 t429 0 0.1f
M1167 t426 nw95 t429 0 nch w=1u l=180n
M1168 t429 t425 0 0 nch w=1u l=180n
M1169 t427 nw61 vdd vdd pch w=2u l=180n
M1170 t427 t425 vdd vdd pch w=2u l=180n
CT430 t430 0 0.1f
M1171 t427 nw61 t430 0 nch w=1u l=180n
M1172 t430 t425 0 0 nch w=1u l=180n
M1173 nw157 t426 vdd vdd pch w=2u l=180n
M1174 nw157 t427 vdd vdd pch w=2u l=180n
CT431 t431 0 0.1f
M1175 nw157 t426 t431 0 nch w=1u l=180n
M1176 t431 t427 0 0 nch w=1u l=180n
Cnw157 nw157 0 2f
M1177 nw158 nw96 vdd vdd pch w=2u l=180n
M1178 nw158 nw62 vdd vdd pch w=2u l=180n
CT432 t432 0 0.1f
M1179 nw158 nw96 t432 0 nch w=1u l=180n
M1180 t432 nw62 0 0 nch w=1u l=180n
Cnw158 nw158 0 2f
M1181 nw159 nw97 0 0 nch w=1u l=180n
M1182 nw159 nw63 0 0 nch w=1u l=180n
CT433 t433 0 0.1f
M1183 t433 nw97 vdd vdd pch w=2u l=180n
M1184 nw159 nw63 t433 vdd pch w=2u l=180n
Cnw159 nw159 0 2f
CT434 t434 0 0.1f
M1185 t434 nw98 vdd vdd pch w=2u l=180n
M1186 t434 nw64 vdd vdd pch w=2u l=180n
CT435 t435 0 0.1f
M1187 t434 nw98 t435 0 nch w=1u l=180n
M1188 t435 nw64 0 0 nch w=1u l=180n
M1189 nw160 t434 vdd vdd pch w=2u l=180n
M1190 nw160 t434 0 0 nch w=1u l=180n
Cnw160 nw160 0 2f
CT436 t436 0 0.1f
M1191 t436 nw99 0 0 nch w=1u l=180n
M1192 t436 nw65 0 0 nch w=1u l=180n
CT437 t437 0 0.1f
M1193 t437 nw99 vdd vdd pch w=2u l=180n
M1194 t436 nw65 t437 vdd pch w=2u l=180n
M1195 nw161 t436 vdd vdd pch w=2u l=180n
M1196 nw161 t436 0 0 nch w=1u l=180n
Cnw161 nw161 0 2f
CT438 t438 0 0.1f
CT439 t439 0 0.1f
CT440 t440 0 0.1f
M1197 t438 nw100 vdd vdd pch w=2u l=180n
M1198 t438 nw66 vdd vdd pch w=2u l=180n
CT441 t441 0 0.1f
M1199 t438 nw100 t441 0 nch w=1u l=180n
M1200 t441 nw66 0 0 nch w=1u l=180n
M1201 t439 nw100 vdd vdd pch w=2u l=180n
M1202 t439 t438 vdd vdd pch w=2u l=180n
CT442 t442 0 0.1f
M1203 t439 nw100 t442 0 nch w=1u l=180n
M1204 t442 t438 0 0 nch w=1u l=180n
M1205 t440 nw66 vdd vdd pch w=2u l=180n
M1206 t440 t438 vdd vdd pch w=2u l=180n
CT443 t443 0 0.1f
M1207 t440 nw66 t443 0 nch w=1u l=180n
M1208 t443 t438 0 0 nch w=1u l=180n
M1209 nw162 t439 vdd vdd pch w=2u l=180n
M1210 nw162 t440 vdd vdd pch w=2u l=180n
CT444 t444 0 0.1f
M1211 nw162 t439 t444 0 nch w=1u l=180n
M1212 t444 t440 0 0 nch w=1u l=180n
Cnw162 nw162 0 2f
M1213 nw163 nw101 vdd vdd pch w=2u l=180n
M1214 nw163 nw67 vdd vdd pch w=2u l=180n
CT445 t445 0 0.1f
M1215 nw163 nw101 t445 0 nch w=1u l=180n
M1216 t445 nw67 0 0 nch w=1u l=180n
Cnw163 nw163 0 2f
M1217 nw164 nw102 0 0 nch w=1u l=180n
M1218 nw164 nw68 0 0 nch w=1u l=180n
CT446 t446 0 0.1f
M1219 t446 nw102 vdd vdd pch w=2u l=180n
M1220 nw164 nw68 t446 vdd pch w=2u l=180n
Cnw164 nw164 0 2f
CT447 t447 0 0.1f
M1221 t447 nw103 vdd vdd pch w=2u l=180n
M1222 t447 nw69 vdd vdd pch w=2u l=180n
CT448 t448 0 0.1f
M1223 t447 nw103 t448 0 nch w=1u l=180n
M1224 t448 nw69 0 0 nch w=1u l=180n
M1225 nw165 t447 vdd vdd pch w=2u l=180n
M1226 nw165 t447 0 0 nch w=1u l=180n
Cnw165 nw165 0 2f
CT449 t449 0 0.1f
M1227 t449 nw104 0 0 nch w=1u l=180n
M1228 t449 nw70 0 0 nch w=1u l=180n
CT450 t450 0 0.1f
M1229 t450 nw104 vdd vdd pch w=2u l=180n
M1230 t449 nw70 t450 vdd pch w=2u l=180n
M1231 nw166 t449 vdd vdd pch w=2u l=180n
M1232 nw166 t449 0 0 nch w=1u l=180n
Cnw166 nw166 0 2f
CT451 t451 0 0.1f
CT452 t452 0 0.1f
CT453 t453 0 0.1f
M1233 t451 nw105 vdd vdd pch w=2u l=180n
M1234 t451 nw71 vdd vdd pch w=2u l=180n
CT454 t454 0 0.1f
M1235 t451 nw105 t454 0 nch w=1u l=180n
M1236 t454 nw71 0 0 nch w=1u l=180n
M1237 t452 nw105 vdd vdd pch w=2u l=180n
M1238 t452 t451 vdd vdd pch w=2u l=180n
CT455 t455 0 0.1f
M1239 t452 nw105 t455 0 nch w=1u l=180n
M1240 t455 t451 0 0 nch w=1u l=180n
M1241 t453 nw71 vdd vdd pch w=2u l=180n
M1242 t453 t451 vdd vdd pch w=2u l=180n
CT456 t456 0 0.1f
M1243 t453 nw71 t456 0 nch w=1u l=180n
M1244 t456 t451 0 0 nch w=1u l=180n
M1245 nw167 t452 vdd vdd pch w=2u l=180n
M1246 nw167 t453 vdd vdd pch w=2u l=180n
CT457 t457 0 0.1f
M1247 nw167 t452 t457 0 nch w=1u l=180n
M1248 t457 t453 0 0 nch w=1u l=180n
Cnw167 nw167 0 2f
M1249 nw168 nw106 vdd vdd pch w=2u l=180n
M1250 nw168 nw72 vdd vdd pch w=2u l=180n
CT458 t458 0 0.1f
M1251 nw168 nw106 t458 0 nch w=1u l=180n
M1252 t458 nw72 0 0 nch w=1u l=180n
Cnw168 nw168 0 2f
M1253 nw169 nw107 0 0 nch w=1u l=180n
M1254 nw169 nw73 0 0 nch w=1u l=180n
CT459 t459 0 0.1f
M1255 t459 nw107 vdd vdd pch w=2u l=180n
M1256 nw169 nw73 t459 vdd pch w=2u l=180n
Cnw169 nw169 0 2f
CT460 t460 0 0.1f
M1257 t460 nw108 vdd vdd pch w=2u l=180n
M1258 t460 nw74 vdd vdd pch w=2u l=180n
CT461 t461 0 0.1f
M1259 t460 nw108 t461 0 nch w=1u l=180n
M1260 t461 nw74 0 0 nch w=1u l=180n
M1261 nw170 t460 vdd vdd pch w=2u l=180n
M1262 nw170 t460 0 0 nch w=1u l=180n
Cnw170 nw170 0 2f
CT462 t462 0 0.1f
M1263 t462 nw109 0 0 nch w=1u l=180n
M1264 t462 nw75 0 0 nch w=1u l=180n
CT463 t463 0 0.1f
M1265 t463 nw109 vdd vdd pch w=2u l=180n
M1266 t462 nw75 t463 vdd pch w=2u l=180n
M1267 nw171 t462 vdd vdd pch w=2u l=180n
M1268 nw171 t462 0 0 nch w=1u l=180n
Cnw171 nw171 0 2f
CT464 t464 0 0.1f
CT465 t465 0 0.1f
CT466 t466 0 0.1f
M1269 t464 nw110 vdd vdd pch w=2u l=180n
M1270 t464 nw76 vdd vdd pch w=2u l=180n
CT467 t467 0 0.1f
M1271 t464 nw110 t467 0 nch w=1u l=180n
M1272 t467 nw76 0 0 nch w=1u l=180n
M1273 t465 nw110 vdd vdd pch w=2u l=180n
M1274 t465 t464 vdd vdd pch w=2u l=180n
CT468 t468 0 0.1f
M1275 t465 nw110 t468 0 nch w=1u l=180n
M1276 t468 t464 0 0 nch w=1u l=180n
M1277 t466 nw76 vdd vdd pch w=2u l=180n
M1278 t466 t464 vdd vdd pch w=2u l=180n
CT469 t469 0 0.1f
M1279 t466 nw76 t469 0 nch w=1u l=180n
M1280 t469 t464 0 0 nch w=1u l=180n
M1281 nw172 t465 vdd vdd pch w=2u l=180n
M1282 nw172 t466 vdd vdd pch w=2u l=180n
CT470 t470 0 0.1f
M1283 nw172 t465 t470 0 nch w=1u l=180n
M1284 t470 t466 0 0 nch w=1u l=180n
Cnw172 nw172 0 2f
M1285 nw173 nw111 vdd vdd pch w=2u l=180n
M1286 nw173 nw77 vdd vdd pch w=2u l=180n
CT471 t471 0 0.1f
M1287 nw173 nw111 t471 0 nch w=1u l=180n
M1288 t471 nw77 0 0 nch w=1u l=180n
Cnw173 nw173 0 2f
M1289 nw174 nw112 0 0 nch w=1u l=180n
M1290 nw174 nw78 0 0 nch w=1u l=180n
CT472 t472 0 0.1f
M1291 t472 nw112 vdd vdd pch w=2u l=180n
M1292 nw174 nw78 t472 vdd pch w=2u l=180n
Cnw174 nw174 0 2f
CT473 t473 0 0.1f
M1293 t473 nw113 vdd vdd pch w=2u l=180n
M1294 t473 nw79 vdd vdd pch w=2u l=180n
CT474 t474 0 0.1f
M1295 t473 nw113 t474 0 nch w=1u l=180n
M1296 t474 nw79 0 0 nch w=1u l=180n
M1297 nw175 t473 vdd vdd pch w=2u l=180n
M1298 nw175 t473 0 0 nch w=1u l=180n
Cnw175 nw175 0 2f
CT475 t475 0 0.1f
M1299 t475 nw114 0 0 nch w=1u l=180n
M1300 t475 nw80 0 0 nch w=1u l=180n
CT476 t476 0 0.1f
M1301 t476 nw114 vdd vdd pch w=2u l=180n
M1302 t475 nw80 t476 vdd pch w=2u l=180n
M1303 nw176 t475 vdd vdd pch w=2u l=180n
M1304 nw176 t475 0 0 nch w=1u l=180n
Cnw176 nw176 0 2f
CT477 t477 0 0.1f
CT478 t478 0 0.1f
CT479 t479 0 0.1f
M1305 t477 nw115 vdd vdd pch w=2u l=180n
M1306 t477 nw81 vdd vdd pch w=2u l=180n
CT480 t480 0 0.1f
M1307 t477 nw115 t480 0 nch w=1u l=180n
M1308 t480 nw81 0 0 nch w=1u l=180n
M1309 t478 nw115 vdd vdd pch w=2u l=180n
M1310 t478 t477 vdd vdd pch w=2u l=180n
CT481 t481 0 0.1f
M1311 t478 nw115 t481 0 nch w=1u l=180n
M1312 t481 t477 0 0 nch w=1u l=180n
M1313 t479 nw81 vdd vdd pch w=2u l=180n
M1314 t479 t477 vdd vdd pch w=2u l=180n
CT482 t482 0 0.1f
M1315 t479 nw81 t482 0 nch w=1u l=180n
M1316 t482 t477 0 0 nch w=1u l=180n
M1317 nw177 t478 vdd vdd pch w=2u l=180n
M1318 nw177 t479 vdd vdd pch w=2u l=180n
CT483 t483 0 0.1f
M1319 nw177 t478 t483 0 nch w=1u l=180n
M1320 t483 t479 0 0 nch w=1u l=180n
Cnw177 nw177 0 2f
M1321 nw178 nw116 vdd vdd pch w=2u l=180n
M1322 nw178 nw82 vdd vdd pch w=2u l=180n
CT484 t484 0 0.1f
M1323 nw178 nw116 t484 0 nch w=1u l=180n
M1324 t484 nw82 0 0 nch w=1u l=180n
Cnw178 nw178 0 2f
M1325 nw179 nw117 0 0 nch w=1u l=180n
M1326 nw179 nw83 0 0 nch w=1u l=180n
CT485 t485 0 0.1f
M1327 t485 nw117 vdd vdd pch w=2u l=180n
M1328 nw179 nw83 t485 vdd pch w=2u l=180n
Cnw179 nw179 0 2f
CT486 t486 0 0.1f
M1329 t486 nw118 vdd vdd pch w=2u l=180n
M1330 t486 nw84 vdd vdd pch w=2u l=180n
CT487 t487 0 0.1f
M1331 t486 nw118 t487 0 nch w=1u l=180n
M1332 t487 nw84 0 0 nch w=1u l=180n
M1333 nw180 t486 vdd vdd pch w=2u l=180n
M1334 nw180 t486 0 0 nch w=1u l=180n
Cnw180 nw180 0 2f
CT488 t488 0 0.1f
M1335 t488 nw119 0 0 nch w=1u l=180n
M1336 t488 nw85 0 0 nch w=1u l=180n
CT489 t489 0 0.1f
M1337 t489 nw119 vdd vdd pch w=2u l=180n
M1338 t488 nw85 t489 vdd pch w=2u l=180n
M1339 nw181 t488 vdd vdd pch w=2u l=180n
M1340 nw181 t488 0 0 nch w=1u l=180n
Cnw181 nw181 0 2f
CT490 t490 0 0.1f
CT491 t491 0 0.1f
CT492 t492 0 0.1f
M1341 t490 nw120 vdd vdd pch w=2u l=180n
M1342 t490 nw86 vdd vdd pch w=2u l=180n
CT493 t493 0 0.1f
M1343 t490 nw120 t493 0 nch w=1u l=180n
M1344 t493 nw86 0 0 nch w=1u l=180n
M1345 t491 nw120 vdd vdd pch w=2u l=180n
M1346 t491 t490 vdd vdd pch w=2u l=180n
CT494 t494 0 0.1f
M1347 t491 nw120 t494 0 nch w=1u l=180n
M1348 t494 t490 0 0 nch w=1u l=180n
M1349 t492 nw86 vdd vdd pch w=2u l=180n
M1350 t492 t490 vdd vdd pch w=2u l=180n
CT495 t495 0 0.1f
M1351 t492 nw86 t495 0 nch w=1u l=180n
M1352 t495 t490 0 0 nch w=1u l=180n
M1353 nw182 t491 vdd vdd pch w=2u l=180n
M1354 nw182 t492 vdd vdd pch w=2u l=180n
CT496 t496 0 0.1f
M1355 nw182 t491 t496 0 nch w=1u l=180n
M1356 t496 t492 0 0 nch w=1u l=180n
Cnw182 nw182 0 2f
M1357 nw183 nw121 vdd vdd pch w=2u l=180n
M1358 nw183 nw87 vdd vdd pch w=2u l=180n
CT497 t497 0 0.1f
M1359 nw183 nw121 t497 0 nch w=1u l=180n
M1360 t497 nw87 0 0 nch w=1u l=180n
Cnw183 nw183 0 2f
M1361 nw184 nw122 0 0 nch w=1u l=180n
M1362 nw184 nw88 0 0 nch w=1u l=180n
CT498 t498 0 0.1f
M1363 t498 nw122 vdd vdd pch w=2u l=180n
M1364 nw184 nw88 t498 vdd pch w=2u l=180n
Cnw184 nw184 0 2f
CT499 t499 0 0.1f
M1365 t499 nw123 vdd vdd pch w=2u l=180n
M1366 t499 nw89 vdd vdd pch w=2u l=180n
CT500 t500 0 0.1f
M1367 t499 nw123 t500 0 nch w=1u l=180n
M1368 t500 nw89 0 0 nch w=1u l=180n
M1369 nw185 t499 vdd vdd pch w=2u l=180n
M1370 nw185 t499 0 0 nch w=1u l=180n
Cnw185 nw185 0 2f
CT501 t501 0 0.1f
M1371 t501 nw124 0 0 nch w=1u l=180n
M1372 t501 nw90 0 0 nch w=1u l=180n
CT502 t502 0 0.1f
M1373 t502 nw124 vdd vdd pch w=2u l=180n
M1374 t501 nw90 t502 vdd pch w=2u l=180n
M1375 nw186 t501 vdd vdd pch w=2u l=180n
M1376 nw186 t501 0 0 nch w=1u l=180n
Cnw186 nw186 0 2f
CT503 t503 0 0.1f
CT504 t504 0 0.1f
CT505 t505 0 0.1f
M1377 t503 nw125 vdd vdd pch w=2u l=180n
M1378 t503 nw91 vdd vdd pch w=2u l=180n
CT506 t506 0 0.1f
M1379 t503 nw125 t506 0 nch w=1u l=180n
M1380 t506 nw91 0 0 nch w=1u l=180n
M1381 t504 nw125 vdd vdd pch w=2u l=180n
M1382 t504 t503 vdd vdd pch w=2u l=180n
CT507 t507 0 0.1f
M1383 t504 nw125 t507 0 nch w=1u l=180n
M1384 t507 t503 0 0 nch w=1u l=180n
M1385 t505 nw91 vdd vdd pch w=2u l=180n
M1386 t505 t503 vdd vdd pch w=2u l=180n
CT508 t508 0 0.1f
M1387 t505 nw91 t508 0 nch w=1u l=180n
M1388 t508 t503 0 0 nch w=1u l=180n
M1389 nw187 t504 vdd vdd pch w=2u l=180n
M1390 nw187 t505 vdd vdd pch w=2u l=180n
CT509 t509 0 0.1f
M1391 nw187 t504 t509 0 nch w=1u l=180n
M1392 t509 t505 0 0 nch w=1u l=180n
Cnw187 nw187 0 2f
M1393 nw188 nw126 vdd vdd pch w=2u l=180n
M1394 nw188 nw92 vdd vdd pch w=2u l=180n
CT510 t510 0 0.1f
M1395 nw188 nw126 t510 0 nch w=1u l=180n
M1396 t510 nw92 0 0 nch w=1u l=180n
Cnw188 nw188 0 2f
M1397 nw189 nw127 0 0 nch w=1u l=180n
M1398 nw189 nw93 0 0 nch w=1u l=180n
CT511 t511 0 0.1f
M1399 t511 nw127 vdd vdd pch w=2u l=180n
M1400 nw189 nw93 t511 vdd pch w=2u l=180n
Cnw189 nw189 0 2f
CT512 t512 0 0.1f
M1401 t512 nw128 vdd vdd pch w=2u l=180n
M1402 t512 nw94 vdd vdd pch w=2u l=180n
CT513 t513 0 0.1f
M1403 t512 nw128 t513 0 nch w=1u l=180n
M1404 t513 nw94 0 0 nch w=1u l=180n
M1405 nw190 t512 vdd vdd pch w=2u l=180n
M1406 nw190 t512 0 0 nch w=1u l=180n
Cnw190 nw190 0 2f
CT514 t514 0 0.1f
M1407 t514 nw129 0 0 nch w=1u l=180n
M1408 t514 nw95 0 0 nch w=1u l=180n
CT515 t515 0 0.1f
M1409 t515 nw129 vdd vdd pch w=2u l=180n
M1410 t514 nw95 t515 vdd pch w=2u l=180n
M1411 nw191 t514 vdd vdd pch w=2u l=180n
M1412 nw191 t514 0 0 nch w=1u l=180n
Cnw191 nw191 0 2f
CT516 t516 0 0.1f
CT517 t517 0 0.1f
CT518 t518 0 0.1f
M1413 t516 nw130 vdd vdd pch w=2u l=180n
M1414 t516 nw96 vdd vdd pch w=2u l=180n
CT519 t519 0 0.1f
M1415 t516 nw130 t519 0 nch w=1u l=180n
M1416 t519 nw96 0 0 nch w=1u l=180n
M1417 t517 nw130 vdd vdd pch w=2u l=180n
M1418 t517 t516 vdd vdd pch w=2u l=180n
CT520 t520 0 0.1f
M1419 t517 nw130 t520 0 nch w=1u l=180n
M1420 t520 t516 0 0 nch w=1u l=180n
M1421 t518 nw96 vdd vdd pch w=2u l=180n
M1422 t518 t516 vdd vdd pch w=2u l=180n
CT521 t521 0 0.1f
M1423 t518 nw96 t521 0 nch w=1u l=180n
M1424 t521 t516 0 0 nch w=1u l=180n
M1425 nw192 t517 vdd vdd pch w=2u l=180n
M1426 nw192 t518 vdd vdd pch w=2u l=180n
CT522 t522 0 0.1f
M1427 nw192 t517 t522 0 nch w=1u l=180n
M1428 t522 t518 0 0 nch w=1u l=180n
Cnw192 nw192 0 2f
M1429 nw193 nw131 vdd vdd pch w=2u l=180n
M1430 nw193 nw97 vdd vdd pch w=2u l=180n
CT523 t523 0 0.1f
M1431 nw193 nw131 t523 0 nch w=1u l=180n
M1432 t523 nw97 0 0 nch w=1u l=180n
Cnw193 nw193 0 2f
M1433 nw194 nw132 0 0 nch w=1u l=180n
M1434 nw194 nw98 0 0 nch w=1u l=180n
CT524 t524 0 0.1f
M1435 t524 nw132 vdd vdd pch w=2u l=180n
M1436 nw194 nw98 t524 vdd pch w=2u l=180n
Cnw194 nw194 0 2f
CT525 t525 0 0.1f
M1437 t525 nw133 vdd vdd pch w=2u l=180n
M1438 t525 nw99 vdd vdd pch w=2u l=180n
CT526 t526 0 0.1f
M1439 t525 nw133 t526 0 nch w=1u l=180n
M1440 t526 nw99 0 0 nch w=1u l=180n
M1441 nw195 t525 vdd vdd pch w=2u l=180n
M1442 nw195 t525 0 0 nch w=1u l=180n
Cnw195 nw195 0 2f
CT527 t527 0 0.1f
M1443 t527 nw134 0 0 nch w=1u l=180n
M1444 t527 nw100 0 0 nch w=1u l=180n
CT528 t528 0 0.1f
M1445 t528 nw134 vdd vdd pch w=2u l=180n
M1446 t527 nw100 t528 vdd pch w=2u l=180n
M1447 nw196 t527 vdd vdd pch w=2u l=180n
M1448 nw196 t527 0 0 nch w=1u l=180n
Cnw196 nw196 0 2f
CT529 t529 0 0.1f
CT530 t530 0 0.1f
CT531 t531 0 0.1f
M1449 t529 nw135 vdd vdd pch w=2u l=180n
M1450 t529 nw101 vdd vdd pch w=2u l=180n
CT532 t532 0 0.1f
M1451 t529 nw135 t532 0 nch w=1u l=180n
M1452 t532 nw101 0 0 nch w=1u l=180n
M1453 t530 nw135 vdd vdd pch w=2u l=180n
M1454 t530 t529 vdd vdd pch w=2u l=180n
CT533 t533 0 0.1f
M1455 t530 nw135 t533 0 nch w=1u l=180n
M1456 t533 t529 0 0 nch w=1u l=180n
M1457 t531 nw101 vdd vdd pch w=2u l=180n
M1458 t531 t529 vdd vdd pch w=2u l=180n
CT534 t534 0 0.1f
M1459 t531 nw101 t534 0 nch w=1u l=180n
M1460 t534 t529 0 0 nch w=1u l=180n
M1461 nw197 t530 vdd vdd pch w=2u l=180n
M1462 nw197 t531 vdd vdd pch w=2u l=180n
CT535 t535 0 0.1f
M1463 nw197 t530 t535 0 nch w=1u l=180n
M1464 t535 t531 0 0 nch w=1u l=180n
Cnw197 nw197 0 2f
M1465 nw198 nw136 vdd vdd pch w=2u l=180n
M1466 nw198 nw102 vdd vdd pch w=2u l=180n
CT536 t536 0 0.1f
M1467 nw198 nw136 t536 0 nch w=1u l=180n
M1468 t536 nw102 0 0 nch w=1u l=180n
Cnw198 nw198 0 2f
M1469 nw199 nw137 0 0 nch w=1u l=180n
M1470 nw199 nw103 0 0 nch w=1u l=180n
CT537 t537 0 0.1f
M1471 t537 nw137 vdd vdd pch w=2u l=180n
M1472 nw199 nw103 t537 vdd pch w=2u l=180n
Cnw199 nw199 0 2f
CT538 t538 0 0.1f
M1473 t538 nw138 vdd vdd pch w=2u l=180n
M1474 t538 nw104 vdd vdd pch w=2u l=180n
CT539 t539 0 0.1f
M1475 t538 nw138 t539 0 nch w=1u l=180n
M1476 t539 nw104 0 0 nch w=1u l=180n
M1477 nw200 t538 vdd vdd pch w=2u l=180n
M1478 nw200 t538 0 0 nch w=1u l=180n
Cnw200 nw200 0 2f
CT540 t540 0 0.1f
M1479 t540 nw139 0 0 nch w=1u l=180n
M1480 t540 nw105 0 0 nch w=1u l=180n
CT541 t541 0 0.1f
M1481 t541 nw139 vdd vdd pch w=2u l=180n
M1482 t540 nw105 t541 vdd pch w=2u l=180n
M1483 nw201 t540 vdd vdd pch w=2u l=180n
M1484 nw201 t540 0 0 nch w=1u l=180n
Cnw201 nw201 0 2f
CT542 t542 0 0.1f
CT543 t543 0 0.1f
CT544 t544 0 0.1f
M1485 t542 nw140 vdd vdd pch w=2u l=180n
M1486 t542 nw106 vdd vdd pch w=2u l=180n
CT545 t545 0 0.1f
M1487 t542 nw140 t545 0 nch w=1u l=180n
M1488 t545 nw106 0 0 nch w=1u l=180n
M1489 t543 nw140 vdd vdd pch w=2u l=180n
M1490 t543 t542 vdd vdd pch w=2u l=180n
CT546 t546 0 0.1f
M1491 t543 nw140 t546 0 nch w=1u l=180n
M1492 t546 t542 0 0 nch w=1u l=180n
M1493 t544 nw106 vdd vdd pch w=2u l=180n
M1494 t544 t542 vdd vdd pch w=2u l=180n
CT547 t547 0 0.1f
M1495 t544 nw106 t547 0 nch w=1u l=180n
M1496 t547 t542 0 0 nch w=1u l=180n
M1497 nw202 t543 vdd vdd pch w=2u l=180n
M1498 nw202 t544 vdd vdd pch w=2u l=180n
CT548 t548 0 0.1f
M1499 nw202 t543 t548 0 nch w=1u l=180n
M1500 t548 t544 0 0 nch w=1u l=180n
Cnw202 nw202 0 2f
M1501 nw203 nw141 vdd vdd pch w=2u l=180n
M1502 nw203 nw107 vdd vdd pch w=2u l=180n
CT549 t549 0 0.1f
M1503 nw203 nw141 t549 0 nch w=1u l=180n
M1504 t549 nw107 0 0 nch w=1u l=180n
Cnw203 nw203 0 2f
M1505 nw204 nw142 0 0 nch w=1u l=180n
M1506 nw204 nw108 0 0 nch w=1u l=180n
CT550 t550 0 0.1f
M1507 t550 nw142 vdd vdd pch w=2u l=180n
M1508 nw204 nw108 t550 vdd pch w=2u l=180n
Cnw204 nw204 0 2f
CT551 t551 0 0.1f
M1509 t551 nw143 vdd vdd pch w=2u l=180n
M1510 t551 nw109 vdd vdd pch w=2u l=180n
CT552 t552 0 0.1f
M1511 t551 nw143 t552 0 nch w=1u l=180n
M1512 t552 nw109 0 0 nch w=1u l=180n
M1513 nw205 t551 vdd vdd pch w=2u l=180n
M1514 nw205 t551 0 0 nch w=1u l=180n
Cnw205 nw205 0 2f
CT553 t553 0 0.1f
M1515 t553 nw144 0 0 nch w=1u l=180n
M1516 t553 nw110 0 0 nch w=1u l=180n
CT554 t554 0 0.1f
M1517 t554 nw144 vdd vdd pch w=2u l=180n
M1518 t553 nw110 t554 vdd pch w=2u l=180n
M1519 nw206 t553 vdd vdd pch w=2u l=180n
M1520 nw206 t553 0 0 nch w=1u l=180n
Cnw206 nw206 0 2f
CT555 t555 0 0.1f
CT556 t556 0 0.1f
CT557 t557 0 0.1f
M1521 t555 nw145 vdd vdd pch w=2u l=180n
M1522 t555 nw111 vdd vdd pch w=2u l=180n
CT558 t558 0 0.1f
M1523 t555 nw145 t558 0 nch w=1u l=180n
M1524 t558 nw111 0 0 nch w=1u l=180n
M1525 t556 nw145 vdd vdd pch w=2u l=180n
M1526 t556 t555 vdd vdd pch w=2u l=180n
CT559 t559 0 0.1f
M1527 t556 nw145 t559 0 nch w=1u l=180n
M1528 t559 t555 0 0 nch w=1u l=180n
M1529 t557 nw111 vdd vdd pch w=2u l=180n
M1530 t557 t555 vdd vdd pch w=2u l=180n
CT560 t560 0 0.1f
M1531 t557 nw111 t560 0 nch w=1u l=180n
M1532 t560 t555 0 0 nch w=1u l=180n
M1533 nw207 t556 vdd vdd pch w=2u l=180n
M1534 nw207 t557 vdd vdd pch w=2u l=180n
CT561 t561 0 0.1f
M1535 nw207 t556 t561 0 nch w=1u l=180n
M1536 t561 t557 0 0 nch w=1u l=180n
Cnw207 nw207 0 2f
M1537 nw208 nw146 vdd vdd pch w=2u l=180n
M1538 nw208 nw112 vdd vdd pch w=2u l=180n
CT562 t562 0 0.1f
M1539 nw208 nw146 t562 0 nch w=1u l=180n
M1540 t562 nw112 0 0 nch w=1u l=180n
Cnw208 nw208 0 2f
M1541 nw209 nw147 0 0 nch w=1u l=180n
M1542 nw209 nw113 0 0 nch w=1u l=180n
CT563 t563 0 0.1f
M1543 t563 nw147 vdd vdd pch w=2u l=180n
M1544 nw209 nw113 t563 vdd pch w=2u l=180n
Cnw209 nw209 0 2f
CT564 t564 0 0.1f
M1545 t564 nw148 vdd vdd pch w=2u l=180n
M1546 t564 nw114 vdd vdd pch w=2u l=180n
CT565 t565 0 0.1f
M1547 t564 nw148 t565 0 nch w=1u l=180n
M1548 t565 nw114 0 0 nch w=1u l=180n
M1549 nw210 t564 vdd vdd pch w=2u l=180n
M1550 nw210 t564 0 0 nch w=1u l=180n
Cnw210 nw210 0 2f
CT566 t566 0 0.1f
M1551 t566 nw149 0 0 nch w=1u l=180n
M1552 t566 nw115 0 0 nch w=1u l=180n
CT567 t567 0 0.1f
M1553 t567 nw149 vdd vdd pch w=2u l=180n
M1554 t566 nw115 t567 vdd pch w=2u l=180n
M1555 nw211 t566 vdd vdd pch w=2u l=180n
M1556 nw211 t566 0 0 nch w=1u l=180n
Cnw211 nw211 0 2f
CT568 t568 0 0.1f
CT569 t569 0 0.1f
CT570 t570 0 0.1f
M1557 t568 nw150 vdd vdd pch w=2u l=180n
M1558 t568 nw116 vdd vdd pch w=2u l=180n
CT571 t571 0 0.1f
M1559 t568 nw150 t571 0 nch w=1u l=180n
M1560 t571 nw116 0 0 nch w=1u l=180n
M1561 t569 nw150 vdd vdd pch w=2u l=180n
M1562 t569 t568 vdd vdd pch w=2u l=180n
CT572 t572 0 0.1f
M1563 t569 nw150 t572 0 nch w=1u l=180n
M1564 t572 t568 0 0 nch w=1u l=180n
M1565 t570 nw116 vdd vdd pch w=2u l=180n
M1566 t570 t568 vdd vdd pch w=2u l=180n
CT573 t573 0 0.1f
M1567 t570 nw116 t573 0 nch w=1u l=180n
M1568 t573 t568 0 0 nch w=1u l=180n
M1569 nw212 t569 vdd vdd pch w=2u l=180n
M1570 nw212 t570 vdd vdd pch w=2u l=180n
CT574 t574 0 0.1f
M1571 nw212 t569 t574 0 nch w=1u l=180n
M1572 t574 t570 0 0 nch w=1u l=180n
Cnw212 nw212 0 2f
M1573 nw213 nw151 vdd vdd pch w=2u l=180n
M1574 nw213 nw117 vdd vdd pch w=2u l=180n
CT575 t575 0 0.1f
M1575 nw213 nw151 t575 0 nch w=1u l=180n
M1576 t575 nw117 0 0 nch w=1u l=180n
Cnw213 nw213 0 2f
M1577 nw214 nw152 0 0 nch w=1u l=180n
M1578 nw214 nw118 0 0 nch w=1u l=180n
CT576 t576 0 0.1f
M1579 t576 nw152 vdd vdd pch w=2u l=180n
M1580 nw214 nw118 t576 vdd pch w=2u l=180n
Cnw214 nw214 0 2f
CT577 t577 0 0.1f
M1581 t577 nw153 vdd vdd pch w=2u l=180n
M1582 t577 nw119 vdd vdd pch w=2u l=180n
CT578 t578 0 0.1f
M1583 t577 nw153 t578 0 nch w=1u l=180n
M1584 t578 nw119 0 0 nch w=1u l=180n
M1585 nw215 t577 vdd vdd pch w=2u l=180n
M1586 nw215 t577 0 0 nch w=1u l=180n
Cnw215 nw215 0 2f
CT579 t579 0 0.1f
M1587 t579 nw154 0 0 nch w=1u l=180n
M1588 t579 nw120 0 0 nch w=1u l=180n
CT580 t580 0 0.1f
M1589 t580 nw154 vdd vdd pch w=2u l=180n
M1590 t579 nw120 t580 vdd pch w=2u l=180n
M1591 nw216 t579 vdd vdd pch w=2u l=180n
M1592 nw216 t579 0 0 nch w=1u l=180n
Cnw216 nw216 0 2f
CT581 t581 0 0.1f
CT582 t582 0 0.1f
CT583 t583 0 0.1f
M1593 t581 nw155 vdd vdd pch w=2u l=180n
M1594 t581 nw121 vdd vdd pch w=2u l=180n
CT584 t584 0 0.1f
M1595 t581 nw155 t584 0 nch w=1u l=180n
M1596 t584 nw121 0 0 nch w=1u l=180n
M1597 t582 nw155 vdd vdd pch w=2u l=180n
M1598 t582 t581 vdd vdd pch w=2u l=180n
CT585 t585 0 0.1f
M1599 t582 nw155 t585 0 nch w=1u l=180n
M1600 t585 t581 0 0 nch w=1u l=180n
M1601 t583 nw121 vdd vdd pch w=2u l=180n
M1602 t583 t581 vdd vdd pch w=2u l=180n
CT586 t586 0 0.1f
M1603 t583 nw121 t586 0 nch w=1u l=180n
M1604 t586 t581 0 0 nch w=1u l=180n
M1605 nw217 t582 vdd vdd pch w=2u l=180n
M1606 nw217 t583 vdd vdd pch w=2u l=180n
CT587 t587 0 0.1f
M1607 nw217 t582 t587 0 nch w=1u l=180n
M1608 t587 t583 0 0 nch w=1u l=180n
Cnw217 nw217 0 2f
M1609 nw218 nw156 vdd vdd pch w=2u l=180n
M1610 nw218 nw122 vdd vdd pch w=2u l=180n
CT588 t588 0 0.1f
M1611 nw218 nw156 t588 0 nch w=1u l=180n
M1612 t588 nw122 0 0 nch w=1u l=180n
Cnw218 nw218 0 2f
M1613 nw219 nw157 0 0 nch w=1u l=180n
M1614 nw219 nw123 0 0 nch w=1u l=180n
CT589 t589 0 0.1f
M1615 t589 nw157 vdd vdd pch w=2u l=180n
M1616 nw219 nw123 t589 vdd pch w=2u l=180n
Cnw219 nw219 0 2f
CT590 t590 0 0.1f
M1617 t590 nw158 vdd vdd pch w=2u l=180n
M1618 t590 nw124 vdd vdd pch w=2u l=180n
CT591 t591 0 0.1f
M1619 t590 nw158 t591 0 nch w=1u l=180n
M1620 t591 nw124 0 0 nch w=1u l=180n
M1621 nw220 t590 vdd vdd pch w=2u l=180n
M1622 nw220 t590 0 0 nch w=1u l=180n
Cnw220 nw220 0 2f
CT592 t592 0 0.1f
M1623 t592 nw159 0 0 nch w=1u l=180n
M1624 t592 nw125 0 0 nch w=1u l=180n
CT593 t593 0 0.1f
M1625 t593 nw159 vdd vdd pch w=2u l=180n
M1626 t592 nw125 t593 vdd pch w=2u l=180n
M1627 nw221 t592 vdd vdd pch w=2u l=180n
M1628 nw221 t592 0 0 nch w=1u l=180n
Cnw221 nw221 0 2f
CT594 t594 0 0.1f
CT595 t595 0 0.1f
CT596 t596 0 0.1f
M1629 t594 nw160 vdd vdd pch w=2u l=180n
M1630 t594 nw126 vdd vdd pch w=2u l=180n
CT597 t597 0 0.1f
M1631 t594 nw160 t597 0 nch w=1u l=180n
M1632 t597 nw126 0 0 nch w=1u l=180n
M1633 t595 nw160 vdd vdd pch w=2u l=180n
M1634 t595 t594 vdd vdd pch w=2u l=180n
CT598 t598 0 0.1f
M1635 t595 nw160 t598 0 nch w=1u l=180n
M1636 t598 t594 0 0 nch w=1u l=180n
M1637 t596 nw126 vdd vdd pch w=2u l=180n
M1638 t596 t594 vdd vdd pch w=2u l=180n
CT599 t599 0 0.1f
M1639 t596 nw126 t599 0 nch w=1u l=180n
M1640 t599 t594 0 0 nch w=1u l=180n
M1641 nw222 t595 vdd vdd pch w=2u l=180n
M1642 nw222 t596 vdd vdd pch w=2u l=180n
CT600 t600 0 0.1f
M1643 nw222 t595 t600 0 nch w=1u l=180n
M1644 t600 t596 0 0 nch w=1u l=180n
Cnw222 nw222 0 2f
M1645 nw223 nw161 vdd vdd pch w=2u l=180n
M1646 nw223 nw127 vdd vdd pch w=2u l=180n
CT601 t601 0 0.1f
M1647 nw223 nw161 t601 0 nch w=1u l=180n
M1648 t601 nw127 0 0 nch w=1u l=180n
Cnw223 nw223 0 2f
M1649 nw224 nw162 0 0 nch w=1u l=180n
M1650 nw224 nw128 0 0 nch w=1u l=180n
CT602 t602 0 0.1f
M1651 t602 nw162 vdd vdd pch w=2u l=180n
M1652 nw224 nw128 t602 vdd pch w=2u l=180n
Cnw224 nw224 0 2f
CT603 t603 0 0.1f
M1653 t603 nw163 vdd vdd pch w=2u l=180n
M1654 t603 nw129 vdd vdd pch w=2u l=180n
CT604 t604 0 0.1f
M1655 t603 nw163 t604 0 nch w=1u l=180n
M1656 t604 nw129 0 0 nch w=1u l=180n
M1657 nw225 t603 vdd vdd pch w=2u l=180n
M1658 nw225 t603 0 0 nch w=1u l=180n
Cnw225 nw225 0 2f
CT605 t605 0 0.1f
M1659 t605 nw164 0 0 nch w=1u l=180n
M1660 t605 nw130 0 0 nch w=1u l=180n
CT606 t606 0 0.1f
M1661 t606 nw164 vdd vdd pch w=2u l=180n
M1662 t605 nw130 t606 vdd pch w=2u l=180n
M1663 nw226 t605 vdd vdd pch w=2u l=180n
M1664 nw226 t605 0 0 nch w=1u l=180n
Cnw226 nw226 0 2f
CT607 t607 0 0.1f
CT608 t608 0 0.1f
CT609 t609 0 0.1f
M1665 t607 nw165 vdd vdd pch w=2u l=180n
M1666 t607 nw131 vdd vdd pch w=2u l=180n
CT610 t610 0 0.1f
M1667 t607 nw165 t610 0 nch w=1u l=180n
M1668 t610 nw131 0 0 nch w=1u l=180n
M1669 t608 nw165 vdd vdd pch w=2u l=180n
M1670 t608 t607 vdd vdd pch w=2u l=180n
CT611 t611 0 0.1f
M1671 t608 nw165 t611 0 nch w=1u l=180n
M1672 t611 t607 0 0 nch w=1u l=180n
M1673 t609 nw131 vdd vdd pch w=2u l=180n
M1674 t609 t607 vdd vdd pch w=2u l=180n
CT612 t612 0 0.1f
M1675 t609 nw131 t612 0 nch w=1u l=180n
M1676 t612 t607 0 0 nch w=1u l=180n
M1677 nw227 t608 vdd vdd pch w=2u l=180n
M1678 nw227 t609 vdd vdd pch w=2u l=180n
CT613 t613 0 0.1f
M1679 nw227 t608 t613 0 nch w=1u l=180n
M1680 t613 t609 0 0 nch w=1u l=180n
Cnw227 nw227 0 2f
M1681 nw228 nw166 vdd vdd pch w=2u l=180n
M1682 nw228 nw132 vdd vdd pch w=2u l=180n
CT614 t614 0 0.1f
M1683 nw228 nw166 t614 0 nch w=1u l=180n
M1684 t614 nw132 0 0 nch w=1u l=180n
Cnw228 nw228 0 2f
M1685 nw229 nw167 0 0 nch w=1u l=180n
M1686 nw229 nw133 0 0 nch w=1u l=180n
CT615 t615 0 0.1f
M1687 t615 nw167 vdd vdd pch w=2u l=180n
M1688 nw229 nw133 t615 vdd pch w=2u l=180n
Cnw229 nw229 0 2f
CT616 t616 0 0.1f
M1689 t616 nw168 vdd vdd pch w=2u l=180n
M1690 t616 nw134 vdd vdd pch w=2u l=180n
CT617 t617 0 0.1f
M1691 t616 nw168 t617 0 nch w=1u l=180n
M1692 t617 nw134 0 0 nch w=1u l=180n
M1693 nw230 t616 vdd vdd pch w=2u l=180n
M1694 nw230 t616 0 0 nch w=1u l=180n
Cnw230 nw230 0 2f
CT618 t618 0 0.1f
M1695 t618 nw169 0 0 nch w=1u l=180n
M1696 t618 nw135 0 0 nch w=1u l=180n
CT619 t619 0 0.1f
M1697 t619 nw169 vdd vdd pch w=2u l=180n
M1698 t618 nw135 t619 vdd pch w=2u l=180n
M1699 nw231 t618 vdd vdd pch w=2u l=180n
M1700 nw231 t618 0 0 nch w=1u l=180n
Cnw231 nw231 0 2f
CT620 t620 0 0.1f
CT621 t621 0 0.1f
CT622 t622 0 0.1f
M1701 t620 nw170 vdd vdd pch w=2u l=180n
M1702 t620 nw136 vdd vdd pch w=2u l=180n
CT623 t623 0 0.1f
M1703 t620 nw170 t623 0 nch w=1u l=180n
M1704 t623 nw136 0 0 nch w=1u l=180n
M1705 t621 nw170 vdd vdd pch w=2u l=180n
M1706 t621 t620 vdd vdd pch w=2u l=180n
CT624 t624 0 0.1f
M1707 t621 nw170 t624 0 nch w=1u l=180n
M1708 t624 t620 0 0 nch w=1u l=180n
M1709 t622 nw136 vdd vdd pch w=2u l=180n
M1710 t622 t620 vdd vdd pch w=2u l=180n
CT625 t625 0 0.1f
M1711 t622 nw136 t625 0 nch w=1u l=180n
M1712 t625 t620 0 0 nch w=1u l=180n
M1713 nw232 t621 vdd vdd pch w=2u l=180n
M1714 nw232 t622 vdd vdd pch w=2u l=180n
CT626 t626 0 0.1f
M1715 nw232 t621 t626 0 nch w=1u l=180n
M1716 t626 t622 0 0 nch w=1u l=180n
Cnw232 nw232 0 2f
M1717 nw233 nw171 vdd vdd pch w=2u l=180n
M1718 nw233 nw137 vdd vdd pch w=2u l=180n
CT627 t627 0 0.1f
M1719 nw233 nw171 t627 0 nch w=1u l=180n
M1720 t627 nw137 0 0 nch w=1u l=180n
Cnw233 nw233 0 2f
M1721 nw234 nw172 0 0 nch w=1u l=180n
M1722 nw234 nw138 0 0 nch w=1u l=180n
CT628 t628 0 0.1f
M1723 t628 nw172 vdd vdd pch w=2u l=180n
M1724 nw234 nw138 t628 vdd pch w=2u l=180n
Cnw234 nw234 0 2f
CT629 t629 0 0.1f
M1725 t629 nw173 vdd vdd pch w=2u l=180n
M1726 t629 nw139 vdd vdd pch w=2u l=180n
CT630 t630 0 0.1f
M1727 t629 nw173 t630 0 nch w=1u l=180n
M1728 t630 nw139 0 0 nch w=1u l=180n
M1729 nw235 t629 vdd vdd pch w=2u l=180n
M1730 nw235 t629 0 0 nch w=1u l=180n
Cnw235 nw235 0 2f
CT631 t631 0 0.1f
M1731 t631 nw174 0 0 nch w=1u l=180n
M1732 t631 nw140 0 0 nch w=1u l=180n
CT632 t632 0 0.1f
M1733 t632 nw174 vdd vdd pch w=2u l=180n
M1734 t631 nw140 t632 vdd pch w=2u l=180n
M1735 nw236 t631 vdd vdd pch w=2u l=180n
M1736 nw236 t631 0 0 nch w=1u l=180n
Cnw236 nw236 0 2f
CT633 t633 0 0.1f
CT634 t634 0 0.1f
CT635 t635 0 0.1f
M1737 t633 nw175 vdd vdd pch w=2u l=180n
M1738 t633 nw141 vdd vdd pch w=2u l=180n
CT636 t636 0 0.1f
M1739 t633 nw175 t636 0 nch w=1u l=180n
M1740 t636 nw141 0 0 nch w=1u l=180n
M1741 t634 nw175 vdd vdd pch w=2u l=180n
M1742 t634 t633 vdd vdd pch w=2u l=180n
CT637 t637 0 0.1f
M1743 t634 nw175 t637 0 nch w=1u l=180n
M1744 t637 t633 0 0 nch w=1u l=180n
M1745 t635 nw141 vdd vdd pch w=2u l=180n
M1746 t635 t633 vdd vdd pch w=2u l=180n
CT638 t638 0 0.1f
M1747 t635 nw141 t638 0 nch w=1u l=180n
M1748 t638 t633 0 0 nch w=1u l=180n
M1749 nw237 t634 vdd vdd pch w=2u l=180n
M1750 nw237 t635 vdd vdd pch w=2u l=180n
CT639 t639 0 0.1f
M1751 nw237 t634 t639 0 nch w=1u l=180n
M1752 t639 t635 0 0 nch w=1u l=180n
Cnw237 nw237 0 2f
M1753 nw238 nw176 vdd vdd pch w=2u l=180n
M1754 nw238 nw142 vdd vdd pch w=2u l=180n
CT640 t640 0 0.1f
M1755 nw238 nw176 t640 0 nch w=1u l=180n
M1756 t640 nw142 0 0 nch w=1u l=180n
Cnw238 nw238 0 2f
M1757 nw239 nw177 0 0 nch w=1u l=180n
M1758 nw239 nw143 0 0 nch w=1u l=180n
CT641 t641 0 0.1f
M1759 t641 nw177 vdd vdd pch w=2u l=180n
M1760 nw239 nw143 t641 vdd pch w=2u l=180n
Cnw239 nw239 0 2f
CT642 t642 0 0.1f
M1761 t642 nw178 vdd vdd pch w=2u l=180n
M1762 t642 nw144 vdd vdd pch w=2u l=180n
CT643 t643 0 0.1f
M1763 t642 nw178 t643 0 nch w=1u l=180n
M1764 t643 nw144 0 0 nch w=1u l=180n
M1765 nw240 t642 vdd vdd pch w=2u l=180n
M1766 nw240 t642 0 0 nch w=1u l=180n
Cnw240 nw240 0 2f
CT644 t644 0 0.1f
M1767 t644 nw179 0 0 nch w=1u l=180n
M1768 t644 nw145 0 0 nch w=1u l=180n
CT645 t645 0 0.1f
M1769 t645 nw179 vdd vdd pch w=2u l=180n
M1770 t644 nw145 t645 vdd pch w=2u l=180n
M1771 nw241 t644 vdd vdd pch w=2u l=180n
M1772 nw241 t644 0 0 nch w=1u l=180n
Cnw241 nw241 0 2f
CT646 t646 0 0.1f
CT647 t647 0 0.1f
CT648 t648 0 0.1f
M1773 t646 nw180 vdd vdd pch w=2u l=180n
M1774 t646 nw146 vdd vdd pch w=2u l=180n
CT649 t649 0 0.1f
M1775 t646 nw180 t649 0 nch w=1u l=180n
M1776 t649 nw146 0 0 nch w=1u l=180n
M1777 t647 nw180 vdd vdd pch w=2u l=180n
M1778 t647 t646 vdd vdd pch w=2u l=180n
CT650 t650 0 0.1f
M1779 t647 nw180 t650 0 nch w=1u l=180n
M1780 t650 t646 0 0 nch w=1u l=180n
M1781 t648 nw146 vdd vdd pch w=2u l=180n
M1782 t648 t646 vdd vdd pch w=2u l=180n
CT651 t651 0 0.1f
M1783 t648 nw146 t651 0 nch w=1u l=180n
M1784 t651 t646 0 0 nch w=1u l=180n
M1785 nw242 t647 vdd vdd pch w=2u l=180n
M1786 nw242 t648 vdd vdd pch w=2u l=180n
CT652 t652 0 0.1f
M1787 nw242 t647 t652 0 nch w=1u l=180n
M1788 t652 t648 0 0 nch w=1u l=180n
Cnw242 nw242 0 2f
M1789 nw243 nw181 vdd vdd pch w=2u l=180n
M1790 nw243 nw147 vdd vdd pch w=2u l=180n
CT653 t653 0 0.1f
M1791 nw243 nw181 t653 0 nch w=1u l=180n
M1792 t653 nw147 0 0 nch w=1u l=180n
Cnw243 nw243 0 2f
M1793 nw244 nw182 0 0 nch w=1u l=180n
M1794 nw244 nw148 0 0 nch w=1u l=180n
CT654 t654 0 0.1f
M1795 t654 nw182 vdd vdd pch w=2u l=180n
M1796 nw244 nw148 t654 vdd pch w=2u l=180n
Cnw244 nw244 0 2f
CT655 t655 0 0.1f
M1797 t655 nw183 vdd vdd pch w=2u l=180n
M1798 t655 nw149 vdd vdd pch w=2u l=180n
CT656 t656 0 0.1f
M1799 t655 nw183 t656 0 nch w=1u l=180n
M1800 t656 nw149 0 0 nch w=1u l=180n
M1801 nw245 t655 vdd vdd pch w=2u l=180n
M1802 nw245 t655 0 0 nch w=1u l=180n
Cnw245 nw245 0 2f
CT657 t657 0 0.1f
M1803 t657 nw184 0 0 nch w=1u l=180n
M1804 t657 nw150 0 0 nch w=1u l=180n
CT658 t658 0 0.1f
M1805 t658 nw184 vdd vdd pch w=2u l=180n
M1806 t657 nw150 t658 vdd pch w=2u l=180n
M1807 nw246 t657 vdd vdd pch w=2u l=180n
M1808 nw246 t657 0 0 nch w=1u l=180n
Cnw246 nw246 0 2f
CT659 t659 0 0.1f
CT660 t660 0 0.1f
CT661 t661 0 0.1f
M1809 t659 nw185 vdd vdd pch w=2u l=180n
M1810 t659 nw151 vdd vdd pch w=2u l=180n
CT662 t662 0 0.1f
M1811 t659 nw185 t662 0 nch w=1u l=180n
M1812 t662 nw151 0 0 nch w=1u l=180n
M1813 t660 nw185 vdd vdd pch w=2u l=180n
M1814 t660 t659 vdd vdd pch w=2u l=180n
CT663 t663 0 0.1f
M1815 t660 nw185 t663 0 nch w=1u l=180n
M1816 t663 t659 0 0 nch w=1u l=180n
M1817 t661 nw151 vdd vdd pch w=2u l=180n
M1818 t661 t659 vdd vdd pch w=2u l=180n
CT664 t664 0 0.1f
M1819 t661 nw151 t664 0 nch w=1u l=180n
M1820 t664 t659 0 0 nch w=1u l=180n
M1821 nw247 t660 vdd vdd pch w=2u l=180n
M1822 nw247 t661 vdd vdd pch w=2u l=180n
CT665 t665 0 0.1f
M1823 nw247 t660 t665 0 nch w=1u l=180n
M1824 t665 t661 0 0 nch w=1u l=180n
Cnw247 nw247 0 2f
M1825 nw248 nw186 vdd vdd pch w=2u l=180n
M1826 nw248 nw152 vdd vdd pch w=2u l=180n
CT666 t666 0 0.1f
M1827 nw248 nw186 t666 0 nch w=1u l=180n
M1828 t666 nw152 0 0 nch w=1u l=180n
Cnw248 nw248 0 2f
M1829 nw249 nw187 0 0 nch w=1u l=180n
M1830 nw249 nw153 0 0 nch w=1u l=180n
CT667 t667 0 0.1f
M1831 t667 nw187 vdd vdd pch w=2u l=180n
M1832 nw249 nw153 t667 vdd pch w=2u l=180n
Cnw249 nw249 0 2f
CT668 t668 0 0.1f
M1833 t668 nw188 vdd vdd pch w=2u l=180n
M1834 t668 nw154 vdd vdd pch w=2u l=180n
CT669 t669 0 0.1f
M1835 t668 nw188 t669 0 nch w=1u l=180n
M1836 t669 nw154 0 0 nch w=1u l=180n
M1837 nw250 t668 vdd vdd pch w=2u l=180n
M1838 nw250 t668 0 0 nch w=1u l=180n
Cnw250 nw250 0 2f
CT670 t670 0 0.1f
M1839 t670 nw189 0 0 nch w=1u l=180n
M1840 t670 nw155 0 0 nch w=1u l=180n
CT671 t671 0 0.1f
M1841 t671 nw189 vdd vdd pch w=2u l=180n
M1842 t670 nw155 t671 vdd pch w=2u l=180n
M1843 nw251 t670 vdd vdd pch w=2u l=180n
M1844 nw251 t670 0 0 nch w=1u l=180n
Cnw251 nw251 0 2f
CT672 t672 0 0.1f
CT673 t673 0 0.1f
CT674 t674 0 0.1f
M1845 t672 nw190 vdd vdd pch w=2u l=180n
M1846 t672 nw156 vdd vdd pch w=2u l=180n
CT675 t675 0 0.1f
M1847 t672 nw190 t675 0 nch w=1u l=180n
M1848 t675 nw156 0 0 nch w=1u l=180n
M1849 t673 nw190 vdd vdd pch w=2u l=180n
M1850 t673 t672 vdd vdd pch w=2u l=180n
CT676 t676 0 0.1f
M1851 t673 nw190 t676 0 nch w=1u l=180n
M1852 t676 t672 0 0 nch w=1u l=180n
M1853 t674 nw156 vdd vdd pch w=2u l=180n
M1854 t674 t672 vdd vdd pch w=2u l=180n
CT677 t677 0 0.1f
M1855 t674 nw156 t677 0 nch w=1u l=180n
M1856 t677 t672 0 0 nch w=1u l=180n
M1857 nw252 t673 vdd vdd pch w=2u l=180n
M1858 nw252 t674 vdd vdd pch w=2u l=180n
CT678 t678 0 0.1f
M1859 nw252 t673 t678 0 nch w=1u l=180n
M1860 t678 t674 0 0 nch w=1u l=180n
Cnw252 nw252 0 2f
M1861 nw253 nw191 vdd vdd pch w=2u l=180n
M1862 nw253 nw157 vdd vdd pch w=2u l=180n
CT679 t679 0 0.1f
M1863 nw253 nw191 t679 0 nch w=1u l=180n
M1864 t679 nw157 0 0 nch w=1u l=180n
Cnw253 nw253 0 2f
M1865 nw254 nw192 0 0 nch w=1u l=180n
M1866 nw254 nw158 0 0 nch w=1u l=180n
CT680 t680 0 0.1f
M1867 t680 nw192 vdd vdd pch w=2u l=180n
M1868 nw254 nw158 t680 vdd pch w=2u l=180n
Cnw254 nw254 0 2f
CT681 t681 0 0.1f
M1869 t681 nw193 vdd vdd pch w=2u l=180n
M1870 t681 nw159 vdd vdd pch w=2u l=180n
CT682 t682 0 0.1f
M1871 t681 nw193 t682 0 nch w=1u l=180n
M1872 t682 nw159 0 0 nch w=1u l=180n
M1873 nw255 t681 vdd vdd pch w=2u l=180n
M1874 nw255 t681 0 0 nch w=1u l=180n
Cnw255 nw255 0 2f
CT683 t683 0 0.1f
M1875 t683 nw194 0 0 nch w=1u l=180n
M1876 t683 nw160 0 0 nch w=1u l=180n
CT684 t684 0 0.1f
M1877 t684 nw194 vdd vdd pch w=2u l=180n
M1878 t683 nw160 t684 vdd pch w=2u l=180n
M1879 nw256 t683 vdd vdd pch w=2u l=180n
M1880 nw256 t683 0 0 nch w=1u l=180n
Cnw256 nw256 0 2f
CT685 t685 0 0.1f
CT686 t686 0 0.1f
CT687 t687 0 0.1f
M1881 t685 nw195 vdd vdd pch w=2u l=180n
M1882 t685 nw161 vdd vdd pch w=2u l=180n
CT688 t688 0 0.1f
M1883 t685 nw195 t688 0 nch w=1u l=180n
M1884 t688 nw161 0 0 nch w=1u l=180n
M1885 t686 nw195 vdd vdd pch w=2u l=180n
M1886 t686 t685 vdd vdd pch w=2u l=180n
CT689 t689 0 0.1f
M1887 t686 nw195 t689 0 nch w=1u l=180n
M1888 t689 t685 0 0 nch w=1u l=180n
M1889 t687 nw161 vdd vdd pch w=2u l=180n
M1890 t687 t685 vdd vdd pch w=2u l=180n
CT690 t690 0 0.1f
M1891 t687 nw161 t690 0 nch w=1u l=180n
M1892 t690 t685 0 0 nch w=1u l=180n
M1893 nw257 t686 vdd vdd pch w=2u l=180n
M1894 nw257 t687 vdd vdd pch w=2u l=180n
CT691 t691 0 0.1f
M1895 nw257 t686 t691 0 nch w=1u l=180n
M1896 t691 t687 0 0 nch w=1u l=180n
Cnw257 nw257 0 2f
M1897 nw258 nw196 vdd vdd pch w=2u l=180n
M1898 nw258 nw162 vdd vdd pch w=2u l=180n
CT692 t692 0 0.1f
M1899 nw258 nw196 t692 0 nch w=1u l=180n
M1900 t692 nw162 0 0 nch w=1u l=180n
Cnw258 nw258 0 2f
M1901 nw259 nw197 0 0 nch w=1u l=180n
M1902 nw259 nw163 0 0 nch w=1u l=180n
CT693 t693 0 0.1f
M1903 t693 nw197 vdd vdd pch w=2u l=180n
M1904 nw259 nw163 t693 vdd pch w=2u l=180n
Cnw259 nw259 0 2f
CT694 t694 0 0.1f
M1905 t694 nw198 vdd vdd pch w=2u l=180n
M1906 t694 nw164 vdd vdd pch w=2u l=180n
CT695 t695 0 0.1f
M1907 t694 nw198 t695 0 nch w=1u l=180n
M1908 t695 nw164 0 0 nch w=1u l=180n
M1909 nw260 t694 vdd vdd pch w=2u l=180n
M1910 nw260 t694 0 0 nch w=1u l=180n
Cnw260 nw260 0 2f
CT696 t696 0 0.1f
M1911 t696 nw199 0 0 nch w=1u l=180n
M1912 t696 nw165 0 0 nch w=1u l=180n
CT697 t697 0 0.1f
M1913 t697 nw199 vdd vdd pch w=2u l=180n
M1914 t696 nw165 t697 vdd pch w=2u l=180n
M1915 nw261 t696 vdd vdd pch w=2u l=180n
M1916 nw261 t696 0 0 nch w=1u l=180n
Cnw261 nw261 0 2f
CT698 t698 0 0.1f
CT699 t699 0 0.1f
CT700 t700 0 0.1f
M1917 t698 nw200 vdd vdd pch w=2u l=180n
M1918 t698 nw166 vdd vdd pch w=2u l=180n
CT701 t701 0 0.1f
M1919 t698 nw200 t701 0 nch w=1u l=180n
M1920 t701 nw166 0 0 nch w=1u l=180n
M1921 t699 nw200 vdd vdd pch w=2u l=180n
M1922 t699 t698 vdd vdd pch w=2u l=180n
CT702 t702 0 0.1f
M1923 t699 nw200 t702 0 nch w=1u l=180n
M1924 t702 t698 0 0 nch w=1u l=180n
M1925 t700 nw166 vdd vdd pch w=2u l=180n
M1926 t700 t698 vdd vdd pch w=2u l=180n
CT703 t703 0 0.1f
M1927 t700 nw166 t703 0 nch w=1u l=180n
M1928 t703 t698 0 0 nch w=1u l=180n
M1929 nw262 t699 vdd vdd pch w=2u l=180n
M1930 nw262 t700 vdd vdd pch w=2u l=180n
CT704 t704 0 0.1f
M1931 nw262 t699 t704 0 nch w=1u l=180n
M1932 t704 t700 0 0 nch w=1u l=180n
Cnw262 nw262 0 2f
M1933 nw263 nw201 vdd vdd pch w=2u l=180n
M1934 nw263 nw167 vdd vdd pch w=2u l=180n
CT705 t705 0 0.1f
M1935 nw263 nw201 t705 0 nch w=1u l=180n
M1936 t705 nw167 0 0 nch w=1u l=180n
Cnw263 nw263 0 2f
M1937 nw264 nw202 0 0 nch w=1u l=180n
M1938 nw264 nw168 0 0 nch w=1u l=180n
CT706 t706 0 0.1f
M1939 t706 nw202 vdd vdd pch w=2u l=180n
M1940 nw264 nw168 t706 vdd pch w=2u l=180n
Cnw264 nw264 0 2f
CT707 t707 0 0.1f
M1941 t707 nw203 vdd vdd pch w=2u l=180n
M1942 t707 nw169 vdd vdd pch w=2u l=180n
CT708 t708 0 0.1f
M1943 t707 nw203 t708 0 nch w=1u l=180n
M1944 t708 nw169 0 0 nch w=1u l=180n
M1945 nw265 t707 vdd vdd pch w=2u l=180n
M1946 nw265 t707 0 0 nch w=1u l=180n
Cnw265 nw265 0 2f
CT709 t709 0 0.1f
M1947 t709 nw204 0 0 nch w=1u l=180n
M1948 t709 nw170 0 0 nch w=1u l=180n
CT710 t710 0 0.1f
M1949 t710 nw204 vdd vdd pch w=2u l=180n
M1950 t709 nw170 t710 vdd pch w=2u l=180n
M1951 nw266 t709 vdd vdd pch w=2u l=180n
M1952 nw266 t709 0 0 nch w=1u l=180n
Cnw266 nw266 0 2f
CT711 t711 0 0.1f
CT712 t712 0 0.1f
CT713 t713 0 0.1f
M1953 t711 nw205 vdd vdd pch w=2u l=180n
M1954 t711 nw171 vdd vdd pch w=2u l=180n
CT714 t714 0 0.1f
M1955 t711 nw205 t714 0 nch w=1u l=180n
M1956 t714 nw171 0 0 nch w=1u l=180n
M1957 t712 nw205 vdd vdd pch w=2u l=180n
M1958 t712 t711 vdd vdd pch w=2u l=180n
CT715 t715 0 0.1f
M1959 t712 nw205 t715 0 nch w=1u l=180n
M1960 t715 t711 0 0 nch w=1u l=180n
M1961 t713 nw171 vdd vdd pch w=2u l=180n
M1962 t713 t711 vdd vdd pch w=2u l=180n
CT716 t716 0 0.1f
M1963 t713 nw171 t716 0 nch w=1u l=180n
M1964 t716 t711 0 0 nch w=1u l=180n
M1965 nw267 t712 vdd vdd pch w=2u l=180n
M1966 nw267 t713 vdd vdd pch w=2u l=180n
CT717 t717 0 0.1f
M1967 nw267 t712 t717 0 nch w=1u l=180n
M1968 t717 t713 0 0 nch w=1u l=180n
Cnw267 nw267 0 2f
M1969 nw268 nw206 vdd vdd pch w=2u l=180n
M1970 nw268 nw172 vdd vdd pch w=2u l=180n
CT718 t718 0 0.1f
M1971 nw268 nw206 t718 0 nch w=1u l=180n
M1972 t718 nw172 0 0 nch w=1u l=180n
Cnw268 nw268 0 2f
M1973 nw269 nw207 0 0 nch w=1u l=180n
M1974 nw269 nw173 0 0 nch w=1u l=180n
CT719 t719 0 0.1f
M1975 t719 nw207 vdd vdd pch w=2u l=180n
M1976 nw269 nw173 t719 vdd pch w=2u l=180n
Cnw269 nw269 0 2f
CT720 t720 0 0.1f
M1977 t720 nw208 vdd vdd pch w=2u l=180n
M1978 t720 nw174 vdd vdd pch w=2u l=180n
CT721 t721 0 0.1f
M1979 t720 nw208 t721 0 nch w=1u l=180n
M1980 t721 nw174 0 0 nch w=1u l=180n
M1981 nw270 t720 vdd vdd pch w=2u l=180n
M1982 nw270 t720 0 0 nch w=1u l=180n
Cnw270 nw270 0 2f
CT722 t722 0 0.1f
M1983 t722 nw209 0 0 nch w=1u l=180n
M1984 t722 nw175 0 0 nch w=1u l=180n
CT723 t723 0 0.1f
M1985 t723 nw209 vdd vdd pch w=2u l=180n
M1986 t722 nw175 t723 vdd pch w=2u l=180n
M1987 nw271 t722 vdd vdd pch w=2u l=180n
M1988 nw271 t722 0 0 nch w=1u l=180n
Cnw271 nw271 0 2f
CT724 t724 0 0.1f
CT725 t725 0 0.1f
CT726 t726 0 0.1f
M1989 t724 nw210 vdd vdd pch w=2u l=180n
M1990 t724 nw176 vdd vdd pch w=2u l=180n
CT727 t727 0 0.1f
M1991 t724 nw210 t727 0 nch w=1u l=180n
M1992 t727 nw176 0 0 nch w=1u l=180n
M1993 t725 nw210 vdd vdd pch w=2u l=180n
M1994 t725 t724 vdd vdd pch w=2u l=180n
CT728 t728 0 0.1f
M1995 t725 nw210 t728 0 nch w=1u l=180n
M1996 t728 t724 0 0 nch w=1u l=180n
M1997 t726 nw176 vdd vdd pch w=2u l=180n
M1998 t726 t724 vdd vdd pch w=2u l=180n
CT729 t729 0 0.1f
M1999 t726 nw176 t729 0 nch w=1u l=180n
M2000 t729 t724 0 0 nch w=1u l=180n
M2001 nw272 t725 vdd vdd pch w=2u l=180n
M2002 nw272 t726 vdd vdd pch w=2u l=180n
CT730 t730 0 0.1f
M2003 nw272 t725 t730 0 nch w=1u l=180n
M2004 t730 t726 0 0 nch w=1u l=180n
Cnw272 nw272 0 2f
M2005 nw273 nw211 vdd vdd pch w=2u l=180n
M2006 nw273 nw177 vdd vdd pch w=2u l=180n
CT731 t731 0 0.1f
M2007 nw273 nw211 t731 0 nch w=1u l=180n
M2008 t731 nw177 0 0 nch w=1u l=180n
Cnw273 nw273 0 2f
M2009 nw274 nw212 0 0 nch w=1u l=180n
M2010 nw274 nw178 0 0 nch w=1u l=180n
CT732 t732 0 0.1f
M2011 t732 nw212 vdd vdd pch w=2u l=180n
M2012 nw274 nw178 t732 vdd pch w=2u l=180n
Cnw274 nw274 0 2f
CT733 t733 0 0.1f
M2013 t733 nw213 vdd vdd pch w=2u l=180n
M2014 t733 nw179 vdd vdd pch w=2u l=180n
CT734 t734 0 0.1f
M2015 t733 nw213 t734 0 nch w=1u l=180n
M2016 t734 nw179 0 0 nch w=1u l=180n
M2017 nw275 t733 vdd vdd pch w=2u l=180n
M2018 nw275 t733 0 0 nch w=1u l=180n
Cnw275 nw275 0 2f
CT735 t735 0 0.1f
M2019 t735 nw214 0 0 nch w=1u l=180n
M2020 t735 nw180 0 0 nch w=1u l=180n
CT736 t736 0 0.1f
M2021 t736 nw214 vdd vdd pch w=2u l=180n
M2022 t735 nw180 t736 vdd pch w=2u l=180n
M2023 nw276 t735 vdd vdd pch w=2u l=180n
M2024 nw276 t735 0 0 nch w=1u l=180n
Cnw276 nw276 0 2f
CT737 t737 0 0.1f
CT738 t738 0 0.1f
CT739 t739 0 0.1f
M2025 t737 nw215 vdd vdd pch w=2u l=180n
M2026 t737 nw181 vdd vdd pch w=2u l=180n
CT740 t740 0 0.1f
M2027 t737 nw215 t740 0 nch w=1u l=180n
M2028 t740 nw181 0 0 nch w=1u l=180n
M2029 t738 nw215 vdd vdd pch w=2u l=180n
M2030 t738 t737 vdd vdd pch w=2u l=180n
CT741 t741 0 0.1f
M2031 t738 nw215 t741 0 nch w=1u l=180n
M2032 t741 t737 0 0 nch w=1u l=180n
M2033 t739 nw181 vdd vdd pch w=2u l=180n
M2034 t739 t737 vdd vdd pch w=2u l=180n
CT742 t742 0 0.1f
M2035 t739 nw181 t742 0 nch w=1u l=180n
M2036 t742 t737 0 0 nch w=1u l=180n
M2037 nw277 t738 vdd vdd pch w=2u l=180n
M2038 nw277 t739 vdd vdd pch w=2u l=180n
CT743 t743 0 0.1f
M2039 nw277 t738 t743 0 nch w=1u l=180n
M2040 t743 t739 0 0 nch w=1u l=180n
Cnw277 nw277 0 2f
M2041 nw278 nw216 vdd vdd pch w=2u l=180n
M2042 nw278 nw182 vdd vdd pch w=2u l=180n
CT744 t744 0 0.1f
M2043 nw278 nw216 t744 0 nch w=1u l=180n
M2044 t744 nw182 0 0 nch w=1u l=180n
Cnw278 nw278 0 2f
M2045 nw279 nw217 0 0 nch w=1u l=180n
M2046 nw279 nw183 0 0 nch w=1u l=180n
CT745 t745 0 0.1f
M2047 t745 nw217 vdd vdd pch w=2u l=180n
M2048 nw279 nw183 t745 vdd pch w=2u l=180n
Cnw279 nw279 0 2f
CT746 t746 0 0.1f
M2049 t746 nw218 vdd vdd pch w=2u l=180n
M2050 t746 nw184 vdd vdd pch w=2u l=180n
CT747 t747 0 0.1f
M2051 t746 nw218 t747 0 nch w=1u l=180n
M2052 t747 nw184 0 0 nch w=1u l=180n
M2053 nw280 t746 vdd vdd pch w=2u l=180n
M2054 nw280 t746 0 0 nch w=1u l=180n
Cnw280 nw280 0 2f
CT748 t748 0 0.1f
M2055 t748 nw219 0 0 nch w=1u l=180n
M2056 t748 nw185 0 0 nch w=1u l=180n
CT749 t749 0 0.1f
M2057 t749 nw219 vdd vdd pch w=2u l=180n
M2058 t748 nw185 t749 vdd pch w=2u l=180n
M2059 nw281 t748 vdd vdd pch w=2u l=180n
M2060 nw281 t748 0 0 nch w=1u l=180n
Cnw281 nw281 0 2f
CT750 t750 0 0.1f
CT751 t751 0 0.1f
CT752 t752 0 0.1f
M2061 t750 nw220 vdd vdd pch w=2u l=180n
M2062 t750 nw186 vdd vdd pch w=2u l=180n
CT753 t753 0 0.1f
M2063 t750 nw220 t753 0 nch w=1u l=180n
M2064 t753 nw186 0 0 nch w=1u l=180n
M2065 t751 nw220 vdd vdd pch w=2u l=180n
M2066 t751 t750 vdd vdd pch w=2u l=180n
CT754 t754 0 0.1f
M2067 t751 nw220 t754 0 nch w=1u l=180n
M2068 t754 t750 0 0 nch w=1u l=180n
M2069 t752 nw186 vdd vdd pch w=2u l=180n
M2070 t752 t750 vdd vdd pch w=2u l=180n
CT755 t755 0 0.1f
M2071 t752 nw186 t755 0 nch w=1u l=180n
M2072 t755 t750 0 0 nch w=1u l=180n
M2073 nw282 t751 vdd vdd pch w=2u l=180n
M2074 nw282 t752 vdd vdd pch w=2u l=180n
CT756 t756 0 0.1f
M2075 nw282 t751 t756 0 nch w=1u l=180n
M2076 t756 t752 0 0 nch w=1u l=180n
Cnw282 nw282 0 2f
M2077 nw283 nw221 vdd vdd pch w=2u l=180n
M2078 nw283 nw187 vdd vdd pch w=2u l=180n
CT757 t757 0 0.1f
M2079 nw283 nw221 t757 0 nch w=1u l=180n
M2080 t757 nw187 0 0 nch w=1u l=180n
Cnw283 nw283 0 2f
M2081 nw284 nw222 0 0 nch w=1u l=180n
M2082 nw284 nw188 0 0 nch w=1u l=180n
CT758 t758 0 0.1f
M2083 t758 nw222 vdd vdd pch w=2u l=180n
M2084 nw284 nw188 t758 vdd pch w=2u l=180n
Cnw284 nw284 0 2f
CT759 t759 0 0.1f
M2085 t759 nw223 vdd vdd pch w=2u l=180n
M2086 t759 nw189 vdd vdd pch w=2u l=180n
CT760 t760 0 0.1f
M2087 t759 nw223 t760 0 nch w=1u l=180n
M2088 t760 nw189 0 0 nch w=1u l=180n
M2089 nw285 t759 vdd vdd pch w=2u l=180n
M2090 nw285 t759 0 0 nch w=1u l=180n
Cnw285 nw285 0 2f
CT761 t761 0 0.1f
M2091 t761 nw224 0 0 nch w=1u l=180n
M2092 t761 nw190 0 0 nch w=1u l=180n
CT762 t762 0 0.1f
M2093 t762 nw224 vdd vdd pch w=2u l=180n
M2094 t761 nw190 t762 vdd pch w=2u l=180n
M2095 nw286 t761 vdd vdd pch w=2u l=180n
M2096 nw286 t761 0 0 nch w=1u l=180n
Cnw286 nw286 0 2f
CT763 t763 0 0.1f
CT764 t764 0 0.1f
CT765 t765 0 0.1f
M2097 t763 nw225 vdd vdd pch w=2u l=180n
M2098 t763 nw191 vdd vdd pch w=2u l=180n
CT766 t766 0 0.1f
M2099 t763 nw225 t766 0 nch w=1u l=180n
M2100 t766 nw191 0 0 nch w=1u l=180n
M2101 t764 nw225 vdd vdd pch w=2u l=180n
M2102 t764 t763 vdd vdd pch w=2u l=180n
CT767 t767 0 0.1f
M2103 t764 nw225 t767 0 nch w=1u l=180n
M2104 t767 t763 0 0 nch w=1u l=180n
M2105 t765 nw191 vdd vdd pch w=2u l=180n
M2106 t765 t763 vdd vdd pch w=2u l=180n
CT768 t768 0 0.1f
M2107 t765 nw191 t768 0 nch w=1u l=180n
M2108 t768 t763 0 0 nch w=1u l=180n
M2109 nw287 t764 vdd vdd pch w=2u l=180n
M2110 nw287 t765 vdd vdd pch w=2u l=180n
CT769 t769 0 0.1f
M2111 nw287 t764 t769 0 nch w=1u l=180n
M2112 t769 t765 0 0 nch w=1u l=180n
Cnw287 nw287 0 2f
M2113 nw288 nw226 vdd vdd pch w=2u l=180n
M2114 nw288 nw192 vdd vdd pch w=2u l=180n
CT770 t770 0 0.1f
M2115 nw288 nw226 t770 0 nch w=1u l=180n
M2116 t770 nw192 0 0 nch w=1u l=180n
Cnw288 nw288 0 2f
M2117 nw289 nw227 0 0 nch w=1u l=180n
M2118 nw289 nw193 0 0 nch w=1u l=180n
CT771 t771 0 0.1f
M2119 t771 nw227 vdd vdd pch w=2u l=180n
M2120 nw289 nw193 t771 vdd pch w=2u l=180n
Cnw289 nw289 0 2f
CT772 t772 0 0.1f
M2121 t772 nw228 vdd vdd pch w=2u l=180n
M2122 t772 nw194 vdd vdd pch w=2u l=180n
CT773 t773 0 0.1f
M2123 t772 nw228 t773 0 nch w=1u l=180n
M2124 t773 nw194 0 0 nch w=1u l=180n
M2125 nw290 t772 vdd vdd pch w=2u l=180n
M2126 nw290 t772 0 0 nch w=1u l=180n
Cnw290 nw290 0 2f
CT774 t774 0 0.1f
M2127 t774 nw229 0 0 nch w=1u l=180n
M2128 t774 nw195 0 0 nch w=1u l=180n
CT775 t775 0 0.1f
M2129 t775 nw229 vdd vdd pch w=2u l=180n
M2130 t774 nw195 t775 vdd pch w=2u l=180n
M2131 nw291 t774 vdd vdd pch w=2u l=180n
M2132 nw291 t774 0 0 nch w=1u l=180n
Cnw291 nw291 0 2f
CT776 t776 0 0.1f
CT777 t777 0 0.1f
CT778 t778 0 0.1f
M2133 t776 nw230 vdd vdd pch w=2u l=180n
M2134 t776 nw196 vdd vdd pch w=2u l=180n
CT779 t779 0 0.1f
M2135 t776 nw230 t779 0 nch w=1u l=180n
M2136 t779 nw196 0 0 nch w=1u l=180n
M2137 t777 nw230 vdd vdd pch w=2u l=180n
M2138 t777 t776 vdd vdd pch w=2u l=180n
CT780 t780 0 0.1f
M2139 t777 nw230 t780 0 nch w=1u l=180n
M2140 t780 t776 0 0 nch w=1u l=180n
M2141 t778 nw196 vdd vdd pch w=2u l=180n
M2142 t778 t776 vdd vdd pch w=2u l=180n
CT781 t781 0 0.1f
M2143 t778 nw196 t781 0 nch w=1u l=180n
M2144 t781 t776 0 0 nch w=1u l=180n
M2145 nw292 t777 vdd vdd pch w=2u l=180n
M2146 nw292 t778 vdd vdd pch w=2u l=180n
CT782 t782 0 0.1f
M2147 nw292 t777 t782 0 nch w=1u l=180n
M2148 t782 t778 0 0 nch w=1u l=180n
Cnw292 nw292 0 2f
M2149 nw293 nw231 vdd vdd pch w=2u l=180n
M2150 nw293 nw197 vdd vdd pch w=2u l=180n
CT783 t783 0 0.1f
M2151 nw293 nw231 t783 0 nch w=1u l=180n
M2152 t783 nw197 0 0 nch w=1u l=180n
Cnw293 nw293 0 2f
M2153 nw294 nw232 0 0 nch w=1u l=180n
M2154 nw294 nw198 0 0 nch w=1u l=180n
CT784 t784 0 0.1f
M2155 t784 nw232 vdd vdd pch w=2u l=180n
M2156 nw294 nw198 t784 vdd pch w=2u l=180n
Cnw294 nw294 0 2f
CT785 t785 0 0.1f
M2157 t785 nw233 vdd vdd pch w=2u l=180n
M2158 t785 nw199 vdd vdd pch w=2u l=180n
CT786 t786 0 0.1f
M2159 t785 nw233 t786 0 nch w=1u l=180n
M2160 t786 nw199 0 0 nch w=1u l=180n
M2161 nw295 t785 vdd vdd pch w=2u l=180n
M2162 nw295 t785 0 0 nch w=1u l=180n
Cnw295 nw295 0 2f
CT787 t787 0 0.1f
M2163 t787 nw234 0 0 nch w=1u l=180n
M2164 t787 nw200 0 0 nch w=1u l=180n
CT788 t788 0 0.1f
M2165 t788 nw234 vdd vdd pch w=2u l=180n
M2166 t787 nw200 t788 vdd pch w=2u l=180n
M2167 nw296 t787 vdd vdd pch w=2u l=180n
M2168 nw296 t787 0 0 nch w=1u l=180n
Cnw296 nw296 0 2f
CT789 t789 0 0.1f
CT790 t790 0 0.1f
CT791 t791 0 0.1f
M2169 t789 nw235 vdd vdd pch w=2u l=180n
M2170 t789 nw201 vdd vdd pch w=2u l=180n
CT792 t792 0 0.1f
M2171 t789 nw235 t792 0 nch w=1u l=180n
M2172 t792 nw201 0 0 nch w=1u l=180n
M2173 t790 nw235 vdd vdd pch w=2u l=180n
M2174 t790 t789 vdd vdd pch w=2u l=180n
CT793 t793 0 0.1f
M2175 t790 nw235 t793 0 nch w=1u l=180n
M2176 t793 t789 0 0 nch w=1u l=180n
M2177 t791 nw201 vdd vdd pch w=2u l=180n
M2178 t791 t789 vdd vdd pch w=2u l=180n
CT794 t794 0 0.1f
M2179 t791 nw201 t794 0 nch w=1u l=180n
M2180 t794 t789 0 0 nch w=1u l=180n
M2181 nw297 t790 vdd vdd pch w=2u l=180n
M2182 nw297 t791 vdd vdd pch w=2u l=180n
CT795 t795 0 0.1f
M2183 nw297 t790 t795 0 nch w=1u l=180n
M2184 t795 t791 0 0 nch w=1u l=180n
Cnw297 nw297 0 2f
M2185 nw298 nw236 vdd vdd pch w=2u l=180n
M2186 nw298 nw202 vdd vdd pch w=2u l=180n
CT796 t796 0 0.1f
M2187 nw298 nw236 t796 0 nch w=1u l=180n
M2188 t796 nw202 0 0 nch w=1u l=180n
Cnw298 nw298 0 2f
M2189 nw299 nw237 0 0 nch w=1u l=180n
M2190 nw299 nw203 0 0 nch w=1u l=180n
CT797 t797 0 0.1f
M2191 t797 nw237 vdd vdd pch w=2u l=180n
M2192 nw299 nw203 t797 vdd pch w=2u l=180n
Cnw299 nw299 0 2f
CT798 t798 0 0.1f
M2193 t798 nw238 vdd vdd pch w=2u l=180n
M2194 t798 nw204 vdd vdd pch w=2u l=180n
CT799 t799 0 0.1f
M2195 t798 nw238 t799 0 nch w=1u l=180n
M2196 t799 nw204 0 0 nch w=1u l=180n
M2197 nw300 t798 vdd vdd pch w=2u l=180n
M2198 nw300 t798 0 0 nch w=1u l=180n
Cnw300 nw300 0 2f
CT800 t800 0 0.1f
M2199 t800 nw239 0 0 nch w=1u l=180n
M2200 t800 nw205 0 0 nch w=1u l=180n
CT801 t801 0 0.1f
M2201 t801 nw239 vdd vdd pch w=2u l=180n
M2202 t800 nw205 t801 vdd pch w=2u l=180n
M2203 nw301 t800 vdd vdd pch w=2u l=180n
M2204 nw301 t800 0 0 nch w=1u l=180n
Cnw301 nw301 0 2f
CT802 t802 0 0.1f
CT803 t803 0 0.1f
CT804 t804 0 0.1f
M2205 t802 nw240 vdd vdd pch w=2u l=180n
M2206 t802 nw206 vdd vdd pch w=2u l=180n
CT805 t805 0 0.1f
M2207 t802 nw240 t805 0 nch w=1u l=180n
M2208 t805 nw206 0 0 nch w=1u l=180n
M2209 t803 nw240 vdd vdd pch w=2u l=180n
M2210 t803 t802 vdd vdd pch w=2u l=180n
CT806 t806 0 0.1f
M2211 t803 nw240 t806 0 nch w=1u l=180n
M2212 t806 t802 0 0 nch w=1u l=180n
M2213 t804 nw206 vdd vdd pch w=2u l=180n
M2214 t804 t802 vdd vdd pch w=2u l=180n
CT807 t807 0 0.1f
M2215 t804 nw206 t807 0 nch w=1u l=180n
M2216 t807 t802 0 0 nch w=1u l=180n
M2217 nw302 t803 vdd vdd pch w=2u l=180n
M2218 nw302 t804 vdd vdd pch w=2u l=180n
CT808 t808 0 0.1f
M2219 nw302 t803 t808 0 nch w=1u l=180n
M2220 t808 t804 0 0 nch w=1u l=180n
Cnw302 nw302 0 2f
M2221 nw303 nw241 vdd vdd pch w=2u l=180n
M2222 nw303 nw207 vdd vdd pch w=2u l=180n
CT809 t809 0 0.1f
M2223 nw303 nw241 t809 0 nch w=1u l=180n
M2224 t809 nw207 0 0 nch w=1u l=180n
Cnw303 nw303 0 2f
M2225 nw304 nw242 0 0 nch w=1u l=180n
M2226 nw304 nw208 0 0 nch w=1u l=180n
CT810 t810 0 0.1f
M2227 t810 nw242 vdd vdd pch w=2u l=180n
M2228 nw304 nw208 t810 vdd pch w=2u l=180n
Cnw304 nw304 0 2f
CT811 t811 0 0.1f
M2229 t811 nw243 vdd vdd pch w=2u l=180n
M2230 t811 nw209 vdd vdd pch w=2u l=180n
CT812 t812 0 0.1f
M2231 t811 nw243 t812 0 nch w=1u l=180n
M2232 t812 nw209 0 0 nch w=1u l=180n
M2233 nw305 t811 vdd vdd pch w=2u l=180n
M2234 nw305 t811 0 0 nch w=1u l=180n
Cnw305 nw305 0 2f
CT813 t813 0 0.1f
M2235 t813 nw244 0 0 nch w=1u l=180n
M2236 t813 nw210 0 0 nch w=1u l=180n
CT814 t814 0 0.1f
M2237 t814 nw244 vdd vdd pch w=2u l=180n
M2238 t813 nw210 t814 vdd pch w=2u l=180n
M2239 nw306 t813 vdd vdd pch w=2u l=180n
M2240 nw306 t813 0 0 nch w=1u l=180n
Cnw306 nw306 0 2f
CT815 t815 0 0.1f
CT816 t816 0 0.1f
CT817 t817 0 0.1f
M2241 t815 nw245 vdd vdd pch w=2u l=180n
M2242 t815 nw211 vdd vdd pch w=2u l=180n
CT818 t818 0 0.1f
M2243 t815 nw245 t818 0 nch w=1u l=180n
M2244 t818 nw211 0 0 nch w=1u l=180n
M2245 t816 nw245 vdd vdd pch w=2u l=180n
M2246 t816 t815 vdd vdd pch w=2u l=180n
CT819 t819 0 0.1f
M2247 t816 nw245 t819 0 nch w=1u l=180n
M2248 t819 t815 0 0 nch w=1u l=180n
M2249 t817 nw211 vdd vdd pch w=2u l=180n
M2250 t817 t815 vdd vdd pch w=2u l=180n
CT820 t820 0 0.1f
M2251 t817 nw211 t820 0 nch w=1u l=180n
M2252 t820 t815 0 0 nch w=1u l=180n
M2253 nw307 t816 vdd vdd pch w=2u l=180n
M2254 nw307 t817 vdd vdd pch w=2u l=180n
CT821 t821 0 0.1f
M2255 nw307 t816 t821 0 nch w=1u l=180n
M2256 t821 t817 0 0 nch w=1u l=180n
Cnw307 nw307 0 2f
M2257 nw308 nw246 vdd vdd pch w=2u l=180n
M2258 nw308 nw212 vdd vdd pch w=2u l=180n
CT822 t822 0 0.1f
M2259 nw308 nw246 t822 0 nch w=1u l=180n
M2260 t822 nw212 0 0 nch w=1u l=180n
Cnw308 nw308 0 2f
M2261 nw309 nw247 0 0 nch w=1u l=180n
M2262 nw309 nw213 0 0 nch w=1u l=180n
CT823 t823 0 0.1f
M2263 t823 nw247 vdd vdd pch w=2u l=180n
M2264 nw309 nw213 t823 vdd pch w=2u l=180n
Cnw309 nw309 0 2f
CT824 t824 0 0.1f
M2265 t824 nw248 vdd vdd pch w=2u l=180n
M2266 t824 nw214 vdd vdd pch w=2u l=180n
CT825 t825 0 0.1f
M2267 t824 nw248 t825 0 nch w=1u l=180n
M2268 t825 nw214 0 0 nch w=1u l=180n
M2269 nw310 t824 vdd vdd pch w=2u l=180n
M2270 nw310 t824 0 0 nch w=1u l=180n
Cnw310 nw310 0 2f
CT826 t826 0 0.1f
M2271 t826 nw249 0 0 nch w=1u l=180n
M2272 t826 nw215 0 0 nch w=1u l=180n
CT827 t827 0 0.1f
M2273 t827 nw249 vdd vdd pch w=2u l=180n
M2274 t826 nw215 t827 vdd pch w=2u l=180n
M2275 nw311 t826 vdd vdd pch w=2u l=180n
M2276 nw311 t826 0 0 nch w=1u l=180n
Cnw311 nw311 0 2f
CT828 t828 0 0.1f
CT829 t829 0 0.1f
CT830 t830 0 0.1f
M2277 t828 nw250 vdd vdd pch w=2u l=180n
M2278 t828 nw216 vdd vdd pch w=2u l=180n
CT831 t831 0 0.1f
M2279 t828 nw250 t831 0 nch w=1u l=180n
M2280 t831 nw216 0 0 nch w=1u l=180n
M2281 t829 nw250 vdd vdd pch w=2u l=180n
M2282 t829 t828 vdd vdd pch w=2u l=180n
CT832 t832 0 0.1f
M2283 t829 nw250 t832 0 nch w=1u l=180n
M2284 t832 t828 0 0 nch w=1u l=180n
M2285 t830 nw216 vdd vdd pch w=2u l=180n
M2286 t830 t828 vdd vdd pch w=2u l=180n
CT833 t833 0 0.1f
M2287 t830 nw216 t833 0 nch w=1u l=180n
M2288 t833 t828 0 0 nch w=1u l=180n
M2289 nw312 t829 vdd vdd pch w=2u l=180n
M2290 nw312 t830 vdd vdd pch w=2u l=180n
CT834 t834 0 0.1f
M2291 nw312 t829 t834 0 nch w=1u l=180n
M2292 t834 t830 0 0 nch w=1u l=180n
Cnw312 nw312 0 2f
M2293 nw313 nw251 vdd vdd pch w=2u l=180n
M2294 nw313 nw217 vdd vdd pch w=2u l=180n
CT835 t835 0 0.1f
M2295 nw313 nw251 t835 0 nch w=1u l=180n
M2296 t835 nw217 0 0 nch w=1u l=180n
Cnw313 nw313 0 2f
M2297 nw314 nw252 0 0 nch w=1u l=180n
M2298 nw314 nw218 0 0 nch w=1u l=180n
CT836 t836 0 0.1f
M2299 t836 nw252 vdd vdd pch w=2u l=180n
M2300 nw314 nw218 t836 vdd pch w=2u l=180n
Cnw314 nw314 0 2f
CT837 t837 0 0.1f
M2301 t837 nw253 vdd vdd pch w=2u l=180n
M2302 t837 nw219 vdd vdd pch w=2u l=180n
CT838 t838 0 0.1f
M2303 t837 nw253 t838 0 nch w=1u l=180n
M2304 t838 nw219 0 0 nch w=1u l=180n
M2305 nw315 t837 vdd vdd pch w=2u l=180n
M2306 nw315 t837 0 0 nch w=1u l=180n
Cnw315 nw315 0 2f
CT839 t839 0 0.1f
M2307 t839 nw254 0 0 nch w=1u l=180n
M2308 t839 nw220 0 0 nch w=1u l=180n
CT840 t840 0 0.1f
M2309 t840 nw254 vdd vdd pch w=2u l=180n
M2310 t839 nw220 t840 vdd pch w=2u l=180n
M2311 nw316 t839 vdd vdd pch w=2u l=180n
M2312 nw316 t839 0 0 nch w=1u l=180n
Cnw316 nw316 0 2f
CT841 t841 0 0.1f
CT842 t842 0 0.1f
CT843 t843 0 0.1f
M2313 t841 nw255 vdd vdd pch w=2u l=180n
M2314 t841 nw221 vdd vdd pch w=2u l=180n
CT844 t844 0 0.1f
M2315 t841 nw255 t844 0 nch w=1u l=180n
M2316 t844 nw221 0 0 nch w=1u l=180n
M2317 t842 nw255 vdd vdd pch w=2u l=180n
M2318 t842 t841 vdd vdd pch w=2u l=180n
CT845 t845 0 0.1f
M2319 t842 nw255 t845 0 nch w=1u l=180n
M2320 t845 t841 0 0 nch w=1u l=180n
M2321 t843 nw221 vdd vdd pch w=2u l=180n
M2322 t843 t841 vdd vdd pch w=2u l=180n
CT846 t846 0 0.1f
M2323 t843 nw221 t846 0 nch w=1u l=180n
M2324 t846 t841 0 0 nch w=1u l=180n
M2325 nw317 t842 vdd vdd pch w=2u l=180n
M2326 nw317 t843 vdd vdd pch w=2u l=180n
CT847 t847 0 0.1f
M2327 nw317 t842 t847 0 nch w=1u l=180n
M2328 t847 t843 0 0 nch w=1u l=180n
Cnw317 nw317 0 2f
M2329 nw318 nw256 vdd vdd pch w=2u l=180n
M2330 nw318 nw222 vdd vdd pch w=2u l=180n
CT848 t848 0 0.1f
M2331 nw318 nw256 t848 0 nch w=1u l=180n
M2332 t848 nw222 0 0 nch w=1u l=180n
Cnw318 nw318 0 2f
M2333 nw319 nw257 0 0 nch w=1u l=180n
M2334 nw319 nw223 0 0 nch w=1u l=180n
CT849 t849 0 0.1f
M2335 t849 nw257 vdd vdd pch w=2u l=180n
M2336 nw319 nw223 t849 vdd pch w=2u l=180n
Cnw319 nw319 0 2f
CT850 t850 0 0.1f
M2337 t850 nw258 vdd vdd pch w=2u l=180n
M2338 t850 nw224 vdd vdd pch w=2u l=180n
CT851 t851 0 0.1f
M2339 t850 nw258 t851 0 nch w=1u l=180n
M2340 t851 nw224 0 0 nch w=1u l=180n
M2341 nw320 t850 vdd vdd pch w=2u l=180n
M2342 nw320 t850 0 0 nch w=1u l=180n
Cnw320 nw320 0 2f
CT852 t852 0 0.1f
M2343 t852 nw259 0 0 nch w=1u l=180n
M2344 t852 nw225 0 0 nch w=1u l=180n
CT853 t853 0 0.1f
M2345 t853 nw259 vdd vdd pch w=2u l=180n
M2346 t852 nw225 t853 vdd pch w=2u l=180n
M2347 nw321 t852 vdd vdd pch w=2u l=180n
M2348 nw321 t852 0 0 nch w=1u l=180n
Cnw321 nw321 0 2f
CT854 t854 0 0.1f
CT855 t855 0 0.1f
CT856 t856 0 0.1f
M2349 t854 nw260 vdd vdd pch w=2u l=180n
M2350 t854 nw226 vdd vdd pch w=2u l=180n
CT857 t857 0 0.1f
M2351 t854 nw260 t857 0 nch w=1u l=180n
M2352 t857 nw226 0 0 nch w=1u l=180n
M2353 t855 nw260 vdd vdd pch w=2u l=180n
M2354 t855 t854 vdd vdd pch w=2u l=180n
CT858 t858 0 0.1f
M2355 t855 nw260 t858 0 nch w=1u l=180n
M2356 t858 t854 0 0 nch w=1u l=180n
M2357 t856 nw226 vdd vdd pch w=2u l=180n
M2358 t856 t854 vdd vdd pch w=2u l=180n
CT859 t859 0 0.1f
M2359 t856 nw226 t859 0 nch w=1u l=180n
M2360 t859 t854 0 0 nch w=1u l=180n
M2361 nw322 t855 vdd vdd pch w=2u l=180n
M2362 nw322 t856 vdd vdd pch w=2u l=180n
CT860 t860 0 0.1f
M2363 nw322 t855 t860 0 nch w=1u l=180n
M2364 t860 t856 0 0 nch w=1u l=180n
Cnw322 nw322 0 2f
M2365 nw323 nw261 vdd vdd pch w=2u l=180n
M2366 nw323 nw227 vdd vdd pch w=2u l=180n
CT861 t861 0 0.1f
M2367 nw323 nw261 t861 0 nch w=1u l=180n
M2368 t861 nw227 0 0 nch w=1u l=180n
Cnw323 nw323 0 2f
M2369 nw324 nw262 0 0 nch w=1u l=180n
M2370 nw324 nw228 0 0 nch w=1u l=180n
CT862 t862 0 0.1f
M2371 t862 nw262 vdd vdd pch w=2u l=180n
M2372 nw324 nw228 t862 vdd pch w=2u l=180n
Cnw324 nw324 0 2f
CT863 t863 0 0.1f
M2373 t863 nw263 vdd vdd pch w=2u l=180n
M2374 t863 nw229 vdd vdd pch w=2u l=180n
CT864 t864 0 0.1f
M2375 t863 nw263 t864 0 nch w=1u l=180n
M2376 t864 nw229 0 0 nch w=1u l=180n
M2377 nw325 t863 vdd vdd pch w=2u l=180n
M2378 nw325 t863 0 0 nch w=1u l=180n
Cnw325 nw325 0 2f
CT865 t865 0 0.1f
M2379 t865 nw264 0 0 nch w=1u l=180n
M2380 t865 nw230 0 0 nch w=1u l=180n
CT866 t866 0 0.1f
M2381 t866 nw264 vdd vdd pch w=2u l=180n
M2382 t865 nw230 t866 vdd pch w=2u l=180n
M2383 nw326 t865 vdd vdd pch w=2u l=180n
M2384 nw326 t865 0 0 nch w=1u l=180n
Cnw326 nw326 0 2f
CT867 t867 0 0.1f
CT868 t868 0 0.1f
CT869 t869 0 0.1f
M2385 t867 nw265 vdd vdd pch w=2u l=180n
M2386 t867 nw231 vdd vdd pch w=2u l=180n
CT870 t870 0 0.1f
M2387 t867 nw265 t870 0 nch w=1u l=180n
M2388 t870 nw231 0 0 nch w=1u l=180n
M2389 t868 nw265 vdd vdd pch w=2u l=180n
M2390 t868 t867 vdd vdd pch w=2u l=180n
CT871 t871 0 0.1f
M2391 t868 nw265 t871 0 nch w=1u l=180n
M2392 t871 t867 0 0 nch w=1u l=180n
M2393 t869 nw231 vdd vdd pch w=2u l=180n
M2394 t869 t867 vdd vdd pch w=2u l=180n
CT872 t872 0 0.1f
M2395 t869 nw231 t872 0 nch w=1u l=180n
M2396 t872 t867 0 0 nch w=1u l=180n
M2397 nw327 t868 vdd vdd pch w=2u l=180n
M2398 nw327 t869 vdd vdd pch w=2u l=180n
CT873 t873 0 0.1f
M2399 nw327 t868 t873 0 nch w=1u l=180n
M2400 t873 t869 0 0 nch w=1u l=180n
Cnw327 nw327 0 2f
M2401 nw328 nw266 vdd vdd pch w=2u l=180n
M2402 nw328 nw232 vdd vdd pch w=2u l=180n
CT874 t874 0 0.1f
M2403 nw328 nw266 t874 0 nch w=1u l=180n
M2404 t874 nw232 0 0 nch w=1u l=180n
Cnw328 nw328 0 2f
M2405 nw329 nw267 0 0 nch w=1u l=180n
M2406 nw329 nw233 0 0 nch w=1u l=180n
CT875 t875 0 0.1f
M2407 t875 nw267 vdd vdd pch w=2u l=180n
M2408 nw329 nw233 t875 vdd pch w=2u l=180n
Cnw329 nw329 0 2f
CT876 t876 0 0.1f
M2409 t876 nw268 vdd vdd pch w=2u l=180n
M2410 t876 nw234 vdd vdd pch w=2u l=180n
CT877 t877 0 0.1f
M2411 t876 nw268 t877 0 nch w=1u l=180n
M2412 t877 nw234 0 0 nch w=1u l=180n
M2413 nw330 t876 vdd vdd pch w=2u l=180n
M2414 nw330 t876 0 0 nch w=1u l=180n
Cnw330 nw330 0 2f
CT878 t878 0 0.1f
M2415 t878 nw269 0 0 nch w=1u l=180n
M2416 t878 nw235 0 0 nch w=1u l=180n
CT879 t879 0 0.1f
M2417 t879 nw269 vdd vdd pch w=2u l=180n
M2418 t878 nw235 t879 vdd pch w=2u l=180n
M2419 nw331 t878 vdd vdd pch w=2u l=180n
M2420 nw331 t878 0 0 nch w=1u l=180n
Cnw331 nw331 0 2f
CT880 t880 0 0.1f
CT881 t881 0 0.1f
CT882 t882 0 0.1f
M2421 t880 nw270 vdd vdd pch w=2u l=180n
M2422 t880 nw236 vdd vdd pch w=2u l=180n
CT883 t883 0 0.1f
M2423 t880 nw270 t883 0 nch w=1u l=180n
M2424 t883 nw236 0 0 nch w=1u l=180n
M2425 t881 nw270 vdd vdd pch w=2u l=180n
M2426 t881 t880 vdd vdd pch w=2u l=180n
CT884 t884 0 0.1f
M2427 t881 nw270 t884 0 nch w=1u l=180n
M2428 t884 t880 0 0 nch w=1u l=180n
M2429 t882 nw236 vdd vdd pch w=2u l=180n
M2430 t882 t880 vdd vdd pch w=2u l=180n
CT885 t885 0 0.1f
M2431 t882 nw236 t885 0 nch w=1u l=180n
M2432 t885 t880 0 0 nch w=1u l=180n
M2433 nw332 t881 vdd vdd pch w=2u l=180n
M2434 nw332 t882 vdd vdd pch w=2u l=180n
CT886 t886 0 0.1f
M2435 nw332 t881 t886 0 nch w=1u l=180n
M2436 t886 t882 0 0 nch w=1u l=180n
Cnw332 nw332 0 2f
M2437 nw333 nw271 vdd vdd pch w=2u l=180n
M2438 nw333 nw237 vdd vdd pch w=2u l=180n
CT887 t887 0 0.1f
M2439 nw333 nw271 t887 0 nch w=1u l=180n
M2440 t887 nw237 0 0 nch w=1u l=180n
Cnw333 nw333 0 2f
M2441 nw334 nw272 0 0 nch w=1u l=180n
M2442 nw334 nw238 0 0 nch w=1u l=180n
CT888 t888 0 0.1f
M2443 t888 nw272 vdd vdd pch w=2u l=180n
M2444 nw334 nw238 t888 vdd pch w=2u l=180n
Cnw334 nw334 0 2f
CT889 t889 0 0.1f
M2445 t889 nw273 vdd vdd pch w=2u l=180n
M2446 t889 nw239 vdd vdd pch w=2u l=180n
CT890 t890 0 0.1f
M2447 t889 nw273 t890 0 nch w=1u l=180n
M2448 t890 nw239 0 0 nch w=1u l=180n
M2449 nw335 t889 vdd vdd pch w=2u l=180n
M2450 nw335 t889 0 0 nch w=1u l=180n
Cnw335 nw335 0 2f
CT891 t891 0 0.1f
M2451 t891 nw274 0 0 nch w=1u l=180n
M2452 t891 nw240 0 0 nch w=1u l=180n
CT892 t892 0 0.1f
M2453 t892 nw274 vdd vdd pch w=2u l=180n
M2454 t891 nw240 t892 vdd pch w=2u l=180n
M2455 nw336 t891 vdd vdd pch w=2u l=180n
M2456 nw336 t891 0 0 nch w=1u l=180n
Cnw336 nw336 0 2f
CT893 t893 0 0.1f
CT894 t894 0 0.1f
CT895 t895 0 0.1f
M2457 t893 nw275 vdd vdd pch w=2u l=180n
M2458 t893 nw241 vdd vdd pch w=2u l=180n
CT896 t896 0 0.1f
M2459 t893 nw275 t896 0 nch w=1u l=180n
M2460 t896 nw241 0 0 nch w=1u l=180n
M2461 t894 nw275 vdd vdd pch w=2u l=180n
M2462 t894 t893 vdd vdd pch w=2u l=180n
CT897 t897 0 0.1f
M2463 t894 nw275 t897 0 nch w=1u l=180n
M2464 t897 t893 0 0 nch w=1u l=180n
M2465 t895 nw241 vdd vdd pch w=2u l=180n
M2466 t895 t893 vdd vdd pch w=2u l=180n
CT898 t898 0 0.1f
M2467 t895 nw241 t898 0 nch w=1u l=180n
M2468 t898 t893 0 0 nch w=1u l=180n
M2469 nw337 t894 vdd vdd pch w=2u l=180n
M2470 nw337 t895 vdd vdd pch w=2u l=180n
CT899 t899 0 0.1f
M2471 nw337 t894 t899 0 nch w=1u l=180n
M2472 t899 t895 0 0 nch w=1u l=180n
Cnw337 nw337 0 2f
M2473 nw338 nw276 vdd vdd pch w=2u l=180n
M2474 nw338 nw242 vdd vdd pch w=2u l=180n
CT900 t900 0 0.1f
M2475 nw338 nw276 t900 0 nch w=1u l=180n
M2476 t900 nw242 0 0 nch w=1u l=180n
Cnw338 nw338 0 2f
M2477 nw339 nw277 0 0 nch w=1u l=180n
M2478 nw339 nw243 0 0 nch w=1u l=180n
CT901 t901 0 0.1f
M2479 t901 nw277 vdd vdd pch w=2u l=180n
M2480 nw339 nw243 t901 vdd pch w=2u l=180n
Cnw339 nw339 0 2f
CT902 t902 0 0.1f
M2481 t902 nw278 vdd vdd pch w=2u l=180n
M2482 t902 nw244 vdd vdd pch w=2u l=180n
CT903 t903 0 0.1f
M2483 t902 nw278 t903 0 nch w=1u l=180n
M2484 t903 nw244 0 0 nch w=1u l=180n
M2485 nw340 t902 vdd vdd pch w=2u l=180n
M2486 nw340 t902 0 0 nch w=1u l=180n
Cnw340 nw340 0 2f
CT904 t904 0 0.1f
M2487 t904 nw279 0 0 nch w=1u l=180n
M2488 t904 nw245 0 0 nch w=1u l=180n
CT905 t905 0 0.1f
M2489 t905 nw279 vdd vdd pch w=2u l=180n
M2490 t904 nw245 t905 vdd pch w=2u l=180n
M2491 nw341 t904 vdd vdd pch w=2u l=180n
M2492 nw341 t904 0 0 nch w=1u l=180n
Cnw341 nw341 0 2f
CT906 t906 0 0.1f
CT907 t907 0 0.1f
CT908 t908 0 0.1f
M2493 t906 nw280 vdd vdd pch w=2u l=180n
M2494 t906 nw246 vdd vdd pch w=2u l=180n
CT909 t909 0 0.1f
M2495 t906 nw280 t909 0 nch w=1u l=180n
M2496 t909 nw246 0 0 nch w=1u l=180n
M2497 t907 nw280 vdd vdd pch w=2u l=180n
M2498 t907 t906 vdd vdd pch w=2u l=180n
CT910 t910 0 0.1f
M2499 t907 nw280 t910 0 nch w=1u l=180n
M2500 t910 t906 0 0 nch w=1u l=180n
M2501 t908 nw246 vdd vdd pch w=2u l=180n
M2502 t908 t906 vdd vdd pch w=2u l=180n
CT911 t911 0 0.1f
M2503 t908 nw246 t911 0 nch w=1u l=180n
M2504 t911 t906 0 0 nch w=1u l=180n
M2505 nw342 t907 vdd vdd pch w=2u l=180n
M2506 nw342 t908 vdd vdd pch w=2u l=180n
CT912 t912 0 0.1f
M2507 nw342 t907 t912 0 nch w=1u l=180n
M2508 t912 t908 0 0 nch w=1u l=180n
Cnw342 nw342 0 2f
M2509 nw343 nw281 vdd vdd pch w=2u l=180n
M2510 nw343 nw247 vdd vdd pch w=2u l=180n
CT913 t913 0 0.1f
M2511 nw343 nw281 t913 0 nch w=1u l=180n
M2512 t913 nw247 0 0 nch w=1u l=180n
Cnw343 nw343 0 2f
M2513 nw344 nw282 0 0 nch w=1u l=180n
M2514 nw344 nw248 0 0 nch w=1u l=180n
CT914 t914 0 0.1f
M2515 t914 nw282 vdd vdd pch w=2u l=180n
M2516 nw344 nw248 t914 vdd pch w=2u l=180n
Cnw344 nw344 0 2f
CT915 t915 0 0.1f
M2517 t915 nw283 vdd vdd pch w=2u l=180n
M2518 t915 nw249 vdd vdd pch w=2u l=180n
CT916 t916 0 0.1f
M2519 t915 nw283 t916 0 nch w=1u l=180n
M2520 t916 nw249 0 0 nch w=1u l=180n
M2521 nw345 t915 vdd vdd pch w=2u l=180n
M2522 nw345 t915 0 0 nch w=1u l=180n
Cnw345 nw345 0 2f
CT917 t917 0 0.1f
M2523 t917 nw284 0 0 nch w=1u l=180n
M2524 t917 nw250 0 0 nch w=1u l=180n
CT918 t918 0 0.1f
M2525 t918 nw284 vdd vdd pch w=2u l=180n
M2526 t917 nw250 t918 vdd pch w=2u l=180n
M2527 nw346 t917 vdd vdd pch w=2u l=180n
M2528 nw346 t917 0 0 nch w=1u l=180n
Cnw346 nw346 0 2f
CT919 t919 0 0.1f
CT920 t920 0 0.1f
CT921 t921 0 0.1f
M2529 t919 nw285 vdd vdd pch w=2u l=180n
M2530 t919 nw251 vdd vdd pch w=2u l=180n
CT922 t922 0 0.1f
M2531 t919 nw285 t922 0 nch w=1u l=180n
M2532 t922 nw251 0 0 nch w=1u l=180n
M2533 t920 nw285 vdd vdd pch w=2u l=180n
M2534 t920 t919 vdd vdd pch w=2u l=180n
CT923 t923 0 0.1f
M2535 t920 nw285 t923 0 nch w=1u l=180n
M2536 t923 t919 0 0 nch w=1u l=180n
M2537 t921 nw251 vdd vdd pch w=2u l=180n
M2538 t921 t919 vdd vdd pch w=2u l=180n
CT924 t924 0 0.1f
M2539 t921 nw251 t924 0 nch w=1u l=180n
M2540 t924 t919 0 0 nch w=1u l=180n
M2541 nw347 t920 vdd vdd pch w=2u l=180n
M2542 nw347 t921 vdd vdd pch w=2u l=180n
CT925 t925 0 0.1f
M2543 nw347 t920 t925 0 nch w=1u l=180n
M2544 t925 t921 0 0 nch w=1u l=180n
Cnw347 nw347 0 2f
M2545 nw348 nw286 vdd vdd pch w=2u l=180n
M2546 nw348 nw252 vdd vdd pch w=2u l=180n
CT926 t926 0 0.1f
M2547 nw348 nw286 t926 0 nch w=1u l=180n
M2548 t926 nw252 0 0 nch w=1u l=180n
Cnw348 nw348 0 2f
M2549 nw349 nw287 0 0 nch w=1u l=180n
M2550 nw349 nw253 0 0 nch w=1u l=180n
CT927 t927 0 0.1f
M2551 t927 nw287 vdd vdd pch w=2u l=180n
M2552 nw349 nw253 t927 vdd pch w=2u l=180n
Cnw349 nw349 0 2f
CT928 t928 0 0.1f
M2553 t928 nw288 vdd vdd pch w=2u l=180n
M2554 t928 nw254 vdd vdd pch w=2u l=180n
CT929 t929 0 0.1f
M2555 t928 nw288 t929 0 nch w=1u l=180n
M2556 t929 nw254 0 0 nch w=1u l=180n
M2557 nw350 t928 vdd vdd pch w=2u l=180n
M2558 nw350 t928 0 0 nch w=1u l=180n
Cnw350 nw350 0 2f
CT930 t930 0 0.1f
M2559 t930 nw289 0 0 nch w=1u l=180n
M2560 t930 nw255 0 0 nch w=1u l=180n
CT931 t931 0 0.1f
M2561 t931 nw289 vdd vdd pch w=2u l=180n
M2562 t930 nw255 t931 vdd pch w=2u l=180n
M2563 nw351 t930 vdd vdd pch w=2u l=180n
M2564 nw351 t930 0 0 nch w=1u l=180n
Cnw351 nw351 0 2f
CT932 t932 0 0.1f
CT933 t933 0 0.1f
CT934 t934 0 0.1f
M2565 t932 nw290 vdd vdd pch w=2u l=180n
M2566 t932 nw256 vdd vdd pch w=2u l=180n
CT935 t935 0 0.1f
M2567 t932 nw290 t935 0 nch w=1u l=180n
M2568 t935 nw256 0 0 nch w=1u l=180n
M2569 t933 nw290 vdd vdd pch w=2u l=180n
M2570 t933 t932 vdd vdd pch w=2u l=180n
CT936 t936 0 0.1f
M2571 t933 nw290 t936 0 nch w=1u l=180n
M2572 t936 t932 0 0 nch w=1u l=180n
M2573 t934 nw256 vdd vdd pch w=2u l=180n
M2574 t934 t932 vdd vdd pch w=2u l=180n
CT937 t937 0 0.1f
M2575 t934 nw256 t937 0 nch w=1u l=180n
M2576 t937 t932 0 0 nch w=1u l=180n
M2577 nw352 t933 vdd vdd pch w=2u l=180n
M2578 nw352 t934 vdd vdd pch w=2u l=180n
CT938 t938 0 0.1f
M2579 nw352 t933 t938 0 nch w=1u l=180n
M2580 t938 t934 0 0 nch w=1u l=180n
Cnw352 nw352 0 2f
M2581 nw353 nw291 vdd vdd pch w=2u l=180n
M2582 nw353 nw257 vdd vdd pch w=2u l=180n
CT939 t939 0 0.1f
M2583 nw353 nw291 t939 0 nch w=1u l=180n
M2584 t939 nw257 0 0 nch w=1u l=180n
Cnw353 nw353 0 2f
M2585 nw354 nw292 0 0 nch w=1u l=180n
M2586 nw354 nw258 0 0 nch w=1u l=180n
CT940 t940 0 0.1f
M2587 t940 nw292 vdd vdd pch w=2u l=180n
M2588 nw354 nw258 t940 vdd pch w=2u l=180n
Cnw354 nw354 0 2f
CT941 t941 0 0.1f
M2589 t941 nw293 vdd vdd pch w=2u l=180n
M2590 t941 nw259 vdd vdd pch w=2u l=180n
CT942 t942 0 0.1f
M2591 t941 nw293 t942 0 nch w=1u l=180n
M2592 t942 nw259 0 0 nch w=1u l=180n
M2593 nw355 t941 vdd vdd pch w=2u l=180n
M2594 nw355 t941 0 0 nch w=1u l=180n
Cnw355 nw355 0 2f
CT943 t943 0 0.1f
M2595 t943 nw294 0 0 nch w=1u l=180n
M2596 t943 nw260 0 0 nch w=1u l=180n
CT944 t944 0 0.1f
M2597 t944 nw294 vdd vdd pch w=2u l=180n
M2598 t943 nw260 t944 vdd pch w=2u l=180n
M2599 nw356 t943 vdd vdd pch w=2u l=180n
M2600 nw356 t943 0 0 nch w=1u l=180n
Cnw356 nw356 0 2f
CT945 t945 0 0.1f
CT946 t946 0 0.1f
CT947 t947 0 0.1f
M2601 t945 nw295 vdd vdd pch w=2u l=180n
M2602 t945 nw261 vdd vdd pch w=2u l=180n
CT948 t948 0 0.1f
M2603 t945 nw295 t948 0 nch w=1u l=180n
M2604 t948 nw261 0 0 nch w=1u l=180n
M2605 t946 nw295 vdd vdd pch w=2u l=180n
M2606 t946 t945 vdd vdd pch w=2u l=180n
CT949 t949 0 0.1f
M2607 t946 nw295 t949 0 nch w=1u l=180n
M2608 t949 t945 0 0 nch w=1u l=180n
M2609 t947 nw261 vdd vdd pch w=2u l=180n
M2610 t947 t945 vdd vdd pch w=2u l=180n
CT950 t950 0 0.1f
M2611 t947 nw261 t950 0 nch w=1u l=180n
M2612 t950 t945 0 0 nch w=1u l=180n
M2613 nw357 t946 vdd vdd pch w=2u l=180n
M2614 nw357 t947 vdd vdd pch w=2u l=180n
CT951 t951 0 0.1f
M2615 nw357 t946 t951 0 nch w=1u l=180n
M2616 t951 t947 0 0 nch w=1u l=180n
Cnw357 nw357 0 2f
M2617 nw358 nw296 vdd vdd pch w=2u l=180n
M2618 nw358 nw262 vdd vdd pch w=2u l=180n
CT952 t952 0 0.1f
M2619 nw358 nw296 t952 0 nch w=1u l=180n
M2620 t952 nw262 0 0 nch w=1u l=180n
Cnw358 nw358 0 2f
M2621 nw359 nw297 0 0 nch w=1u l=180n
M2622 nw359 nw263 0 0 nch w=1u l=180n
CT953 t953 0 0.1f
M2623 t953 nw297 vdd vdd pch w=2u l=180n
M2624 nw359 nw263 t953 vdd pch w=2u l=180n
Cnw359 nw359 0 2f
CT954 t954 0 0.1f
M2625 t954 nw298 vdd vdd pch w=2u l=180n
M2626 t954 nw264 vdd vdd pch w=2u l=180n
CT955 t955 0 0.1f
M2627 t954 nw298 t955 0 nch w=1u l=180n
M2628 t955 nw264 0 0 nch w=1u l=180n
M2629 nw360 t954 vdd vdd pch w=2u l=180n
M2630 nw360 t954 0 0 nch w=1u l=180n
Cnw360 nw360 0 2f
CT956 t956 0 0.1f
M2631 t956 nw299 0 0 nch w=1u l=180n
M2632 t956 nw265 0 0 nch w=1u l=180n
CT957 t957 0 0.1f
M2633 t957 nw299 vdd vdd pch w=2u l=180n
M2634 t956 nw265 t957 vdd pch w=2u l=180n
M2635 nw361 t956 vdd vdd pch w=2u l=180n
M2636 nw361 t956 0 0 nch w=1u l=180n
Cnw361 nw361 0 2f
CT958 t958 0 0.1f
CT959 t959 0 0.1f
CT960 t960 0 0.1f
M2637 t958 nw300 vdd vdd pch w=2u l=180n
M2638 t958 nw266 vdd vdd pch w=2u l=180n
CT961 t961 0 0.1f
M2639 t958 nw300 t961 0 nch w=1u l=180n
M2640 t961 nw266 0 0 nch w=1u l=180n
M2641 t959 nw300 vdd vdd pch w=2u l=180n
M2642 t959 t958 vdd vdd pch w=2u l=180n
CT962 t962 0 0.1f
M2643 t959 nw300 t962 0 nch w=1u l=180n
M2644 t962 t958 0 0 nch w=1u l=180n
M2645 t960 nw266 vdd vdd pch w=2u l=180n
M2646 t960 t958 vdd vdd pch w=2u l=180n
CT963 t963 0 0.1f
M2647 t960 nw266 t963 0 nch w=1u l=180n
M2648 t963 t958 0 0 nch w=1u l=180n
M2649 nw362 t959 vdd vdd pch w=2u l=180n
M2650 nw362 t960 vdd vdd pch w=2u l=180n
CT964 t964 0 0.1f
M2651 nw362 t959 t964 0 nch w=1u l=180n
M2652 t964 t960 0 0 nch w=1u l=180n
Cnw362 nw362 0 2f
M2653 nw363 nw301 vdd vdd pch w=2u l=180n
M2654 nw363 nw267 vdd vdd pch w=2u l=180n
CT965 t965 0 0.1f
M2655 nw363 nw301 t965 0 nch w=1u l=180n
M2656 t965 nw267 0 0 nch w=1u l=180n
Cnw363 nw363 0 2f
M2657 nw364 nw302 0 0 nch w=1u l=180n
M2658 nw364 nw268 0 0 nch w=1u l=180n
CT966 t966 0 0.1f
M2659 t966 nw302 vdd vdd pch w=2u l=180n
M2660 nw364 nw268 t966 vdd pch w=2u l=180n
Cnw364 nw364 0 2f
CT967 t967 0 0.1f
M2661 t967 nw303 vdd vdd pch w=2u l=180n
M2662 t967 nw269 vdd vdd pch w=2u l=180n
CT968 t968 0 0.1f
M2663 t967 nw303 t968 0 nch w=1u l=180n
M2664 t968 nw269 0 0 nch w=1u l=180n
M2665 nw365 t967 vdd vdd pch w=2u l=180n
M2666 nw365 t967 0 0 nch w=1u l=180n
Cnw365 nw365 0 2f
CT969 t969 0 0.1f
M2667 t969 nw304 0 0 nch w=1u l=180n
M2668 t969 nw270 0 0 nch w=1u l=180n
CT970 t970 0 0.1f
M2669 t970 nw304 vdd vdd pch w=2u l=180n
M2670 t969 nw270 t970 vdd pch w=2u l=180n
M2671 nw366 t969 vdd vdd pch w=2u l=180n
M2672 nw366 t969 0 0 nch w=1u l=180n
Cnw366 nw366 0 2f
CT971 t971 0 0.1f
CT972 t972 0 0.1f
CT973 t973 0 0.1f
M2673 t971 nw305 vdd vdd pch w=2u l=180n
M2674 t971 nw271 vdd vdd pch w=2u l=180n
CT974 t974 0 0.1f
M2675 t971 nw305 t974 0 nch w=1u l=180n
M2676 t974 nw271 0 0 nch w=1u l=180n
M2677 t972 nw305 vdd vdd pch w=2u l=180n
M2678 t972 t971 vdd vdd pch w=2u l=180n
CT975 t975 0 0.1f
M2679 t972 nw305 t975 0 nch w=1u l=180n
M2680 t975 t971 0 0 nch w=1u l=180n
M2681 t973 nw271 vdd vdd pch w=2u l=180n
M2682 t973 t971 vdd vdd pch w=2u l=180n
CT976 t976 0 0.1f
M2683 t973 nw271 t976 0 nch w=1u l=180n
M2684 t976 t971 0 0 nch w=1u l=180n
M2685 nw367 t972 vdd vdd pch w=2u l=180n
M2686 nw367 t973 vdd vdd pch w=2u l=180n
CT977 t977 0 0.1f
M2687 nw367 t972 t977 0 nch w=1u l=180n
M2688 t977 t973 0 0 nch w=1u l=180n
Cnw367 nw367 0 2f
M2689 nw368 nw306 vdd vdd pch w=2u l=180n
M2690 nw368 nw272 vdd vdd pch w=2u l=180n
CT978 t978 0 0.1f
M2691 nw368 nw306 t978 0 nch w=1u l=180n
M2692 t978 nw272 0 0 nch w=1u l=180n
Cnw368 nw368 0 2f
M2693 nw369 nw307 0 0 nch w=1u l=180n
M2694 nw369 nw273 0 0 nch w=1u l=180n
CT979 t979 0 0.1f
M2695 t979 nw307 vdd vdd pch w=2u l=180n
M2696 nw369 nw273 t979 vdd pch w=2u l=180n
Cnw369 nw369 0 2f
CT980 t980 0 0.1f
M2697 t980 nw308 vdd vdd pch w=2u l=180n
M2698 t980 nw274 vdd vdd pch w=2u l=180n
CT981 t981 0 0.1f
M2699 t980 nw308 t981 0 nch w=1u l=180n
M2700 t981 nw274 0 0 nch w=1u l=180n
M2701 nw370 t980 vdd vdd pch w=2u l=180n
M2702 nw370 t980 0 0 nch w=1u l=180n
Cnw370 nw370 0 2f
CT982 t982 0 0.1f
M2703 t982 nw309 0 0 nch w=1u l=180n
M2704 t982 nw275 0 0 nch w=1u l=180n
CT983 t983 0 0.1f
M2705 t983 nw309 vdd vdd pch w=2u l=180n
M2706 t982 nw275 t983 vdd pch w=2u l=180n
M2707 nw371 t982 vdd vdd pch w=2u l=180n
M2708 nw371 t982 0 0 nch w=1u l=180n
Cnw371 nw371 0 2f
CT984 t984 0 0.1f
CT985 t985 0 0.1f
CT986 t986 0 0.1f
M2709 t984 nw310 vdd vdd pch w=2u l=180n
M2710 t984 nw276 vdd vdd pch w=2u l=180n
CT987 t987 0 0.1f
M2711 t984 nw310 t987 0 nch w=1u l=180n
M2712 t987 nw276 0 0 nch w=1u l=180n
M2713 t985 nw310 vdd vdd pch w=2u l=180n
M2714 t985 t984 vdd vdd pch w=2u l=180n
CT988 t988 0 0.1f
M2715 t985 nw310 t988 0 nch w=1u l=180n
M2716 t988 t984 0 0 nch w=1u l=180n
M2717 t986 nw276 vdd vdd pch w=2u l=180n
M2718 t986 t984 vdd vdd pch w=2u l=180n
CT989 t989 0 0.1f
M2719 t986 nw276 t989 0 nch w=1u l=180n
M2720 t989 t984 0 0 nch w=1u l=180n
M2721 nw372 t985 vdd vdd pch w=2u l=180n
M2722 nw372 t986 vdd vdd pch w=2u l=180n
CT990 t990 0 0.1f
M2723 nw372 t985 t990 0 nch w=1u l=180n
M2724 t990 t986 0 0 nch w=1u l=180n
Cnw372 nw372 0 2f
M2725 nw373 nw311 vdd vdd pch w=2u l=180n
M2726 nw373 nw277 vdd vdd pch w=2u l=180n
CT991 t991 0 0.1f
M2727 nw373 nw311 t991 0 nch w=1u l=180n
M2728 t991 nw277 0 0 nch w=1u l=180n
Cnw373 nw373 0 2f
M2729 nw374 nw312 0 0 nch w=1u l=180n
M2730 nw374 nw278 0 0 nch w=1u l=180n
CT992 t992 0 0.1f
M2731 t992 nw312 vdd vdd pch w=2u l=180n
M2732 nw374 nw278 t992 vdd pch w=2u l=180n
Cnw374 nw374 0 2f
CT993 t993 0 0.1f
M2733 t993 nw313 vdd vdd pch w=2u l=180n
M2734 t993 nw279 vdd vdd pch w=2u l=180n
CT994 t994 0 0.1f
M2735 t993 nw313 t994 0 nch w=1u l=180n
M2736 t994 nw279 0 0 nch w=1u l=180n
M2737 nw375 t993 vdd vdd pch w=2u l=180n
M2738 nw375 t993 0 0 nch w=1u l=180n
Cnw375 nw375 0 2f
CT995 t995 0 0.1f
M2739 t995 nw314 0 0 nch w=1u l=180n
M2740 t995 nw280 0 0 nch w=1u l=180n
CT996 t996 0 0.1f
M2741 t996 nw314 vdd vdd pch w=2u l=180n
M2742 t995 nw280 t996 vdd pch w=2u l=180n
M2743 nw376 t995 vdd vdd pch w=2u l=180n
M2744 nw376 t995 0 0 nch w=1u l=180n
Cnw376 nw376 0 2f
CT997 t997 0 0.1f
CT998 t998 0 0.1f
CT999 t999 0 0.1f
M2745 t997 nw315 vdd vdd pch w=2u l=180n
M2746 t997 nw281 vdd vdd pch w=2u l=180n
CT1000 t1000 0 0.1f
M2747 t997 nw315 t1000 0 nch w=1u l=180n
M2748 t1000 nw281 0 0 nch w=1u l=180n
M2749 t998 nw315 vdd vdd pch w=2u l=180n
M2750 t998 t997 vdd vdd pch w=2u l=180n
CT1001 t1001 0 0.1f
M2751 t998 nw315 t1001 0 nch w=1u l=180n
M2752 t1001 t997 0 0 nch w=1u l=180n
M2753 t999 nw281 vdd vdd pch w=2u l=180n
M2754 t999 t997 vdd vdd pch w=2u l=180n
CT1002 t1002 0 0.1f
M2755 t999 nw281 t1002 0 nch w=1u l=180n
M2756 t1002 t997 0 0 nch w=1u l=180n
M2757 nw377 t998 vdd vdd pch w=2u l=180n
M2758 nw377 t999 vdd vdd pch w=2u l=180n
CT1003 t1003 0 0.1f
M2759 nw377 t998 t1003 0 nch w=1u l=180n
M2760 t1003 t999 0 0 nch w=1u l=180n
Cnw377 nw377 0 2f
M2761 nw378 nw316 vdd vdd pch w=2u l=180n
M2762 nw378 nw282 vdd vdd pch w=2u l=180n
CT1004 t1004 0 0.1f
M2763 nw378 nw316 t1004 0 nch w=1u l=180n
M2764 t1004 nw282 0 0 nch w=1u l=180n
Cnw378 nw378 0 2f
M2765 nw379 nw317 0 0 nch w=1u l=180n
M2766 nw379 nw283 0 0 nch w=1u l=180n
CT1005 t1005 0 0.1f
M2767 t1005 nw317 vdd vdd pch w=2u l=180n
M2768 nw379 nw283 t1005 vdd pch w=2u l=180n
Cnw379 nw379 0 2f
CT1006 t1006 0 0.1f
M2769 t1006 nw318 vdd vdd pch w=2u l=180n
M2770 t1006 nw284 vdd vdd pch w=2u l=180n
CT1007 t1007 0 0.1f
M2771 t1006 nw318 t1007 0 nch w=1u l=180n
M2772 t1007 nw284 0 0 nch w=1u l=180n
M2773 nw380 t1006 vdd vdd pch w=2u l=180n
M2774 nw380 t1006 0 0 nch w=1u l=180n
Cnw380 nw380 0 2f
CT1008 t1008 0 0.1f
M2775 t1008 nw319 0 0 nch w=1u l=180n
M2776 t1008 nw285 0 0 nch w=1u l=180n
CT1009 t1009 0 0.1f
M2777 t1009 nw319 vdd vdd pch w=2u l=180n
M2778 t1008 nw285 t1009 vdd pch w=2u l=180n
M2779 nw381 t1008 vdd vdd pch w=2u l=180n
M2780 nw381 t1008 0 0 nch w=1u l=180n
Cnw381 nw381 0 2f
CT1010 t1010 0 0.1f
CT1011 t1011 0 0.1f
CT1012 t1012 0 0.1f
M2781 t1010 nw320 vdd vdd pch w=2u l=180n
M2782 t1010 nw286 vdd vdd pch w=2u l=180n
CT1013 t1013 0 0.1f
M2783 t1010 nw320 t1013 0 nch w=1u l=180n
M2784 t1013 nw286 0 0 nch w=1u l=180n
M2785 t1011 nw320 vdd vdd pch w=2u l=180n
M2786 t1011 t1010 vdd vdd pch w=2u l=180n
CT1014 t1014 0 0.1f
M2787 t1011 nw320 t1014 0 nch w=1u l=180n
M2788 t1014 t1010 0 0 nch w=1u l=180n
M2789 t1012 nw286 vdd vdd pch w=2u l=180n
M2790 t1012 t1010 vdd vdd pch w=2u l=180n
CT1015 t1015 0 0.1f
M2791 t1012 nw286 t1015 0 nch w=1u l=180n
M2792 t1015 t1010 0 0 nch w=1u l=180n
M2793 nw382 t1011 vdd vdd pch w=2u l=180n
M2794 nw382 t1012 vdd vdd pch w=2u l=180n
CT1016 t1016 0 0.1f
M2795 nw382 t1011 t1016 0 nch w=1u l=180n
M2796 t1016 t1012 0 0 nch w=1u l=180n
Cnw382 nw382 0 2f
M2797 nw383 nw321 vdd vdd pch w=2u l=180n
M2798 nw383 nw287 vdd vdd pch w=2u l=180n
CT1017 t1017 0 0.1f
M2799 nw383 nw321 t1017 0 nch w=1u l=180n
M2800 t1017 nw287 0 0 nch w=1u l=180n
Cnw383 nw383 0 2f
M2801 nw384 nw322 0 0 nch w=1u l=180n
M2802 nw384 nw288 0 0 nch w=1u l=180n
CT1018 t1018 0 0.1f
M2803 t1018 nw322 vdd vdd pch w=2u l=180n
M2804 nw384 nw288 t1018 vdd pch w=2u l=180n
Cnw384 nw384 0 2f
CT1019 t1019 0 0.1f
M2805 t1019 nw323 vdd vdd pch w=2u l=180n
M2806 t1019 nw289 vdd vdd pch w=2u l=180n
CT1020 t1020 0 0.1f
M2807 t1019 nw323 t1020 0 nch w=1u l=180n
M2808 t1020 nw289 0 0 nch w=1u l=180n
M2809 nw385 t1019 vdd vdd pch w=2u l=180n
M2810 nw385 t1019 0 0 nch w=1u l=180n
Cnw385 nw385 0 2f
CT1021 t1021 0 0.1f
M2811 t1021 nw324 0 0 nch w=1u l=180n
M2812 t1021 nw290 0 0 nch w=1u l=180n
CT1022 t1022 0 0.1f
M2813 t1022 nw324 vdd vdd pch w=2u l=180n
M2814 t1021 nw290 t1022 vdd pch w=2u l=180n
M2815 nw386 t1021 vdd vdd pch w=2u l=180n
M2816 nw386 t1021 0 0 nch w=1u l=180n
Cnw386 nw386 0 2f
CT1023 t1023 0 0.1f
CT1024 t1024 0 0.1f
CT1025 t1025 0 0.1f
M2817 t1023 nw325 vdd vdd pch w=2u l=180n
M2818 t1023 nw291 vdd vdd pch w=2u l=180n
CT1026 t1026 0 0.1f
M2819 t1023 nw325 t1026 0 nch w=1u l=180n
M2820 t1026 nw291 0 0 nch w=1u l=180n
M2821 t1024 nw325 vdd vdd pch w=2u l=180n
M2822 t1024 t1023 vdd vdd pch w=2u l=180n
CT1027 t1027 0 0.1f
M2823 t1024 nw325 t1027 0 nch w=1u l=180n
M2824 t1027 t1023 0 0 nch w=1u l=180n
M2825 t1025 nw291 vdd vdd pch w=2u l=180n
M2826 t1025 t1023 vdd vdd pch w=2u l=180n
CT1028 t1028 0 0.1f
M2827 t1025 nw291 t1028 0 nch w=1u l=180n
M2828 t1028 t1023 0 0 nch w=1u l=180n
M2829 nw387 t1024 vdd vdd pch w=2u l=180n
M2830 nw387 t1025 vdd vdd pch w=2u l=180n
CT1029 t1029 0 0.1f
M2831 nw387 t1024 t1029 0 nch w=1u l=180n
M2832 t1029 t1025 0 0 nch w=1u l=180n
Cnw387 nw387 0 2f
M2833 nw388 nw326 vdd vdd pch w=2u l=180n
M2834 nw388 nw292 vdd vdd pch w=2u l=180n
CT1030 t1030 0 0.1f
M2835 nw388 nw326 t1030 0 nch w=1u l=180n
M2836 t1030 nw292 0 0 nch w=1u l=180n
Cnw388 nw388 0 2f
M2837 nw389 nw327 0 0 nch w=1u l=180n
M2838 nw389 nw293 0 0 nch w=1u l=180n
CT1031 t1031 0 0.1f
M2839 t1031 nw327 vdd vdd pch w=2u l=180n
M2840 nw389 nw293 t1031 vdd pch w=2u l=180n
Cnw389 nw389 0 2f
CT1032 t1032 0 0.1f
M2841 t1032 nw328 vdd vdd pch w=2u l=180n
M2842 t1032 nw294 vdd vdd pch w=2u l=180n
CT1033 t1033 0 0.1f
M2843 t1032 nw328 t1033 0 nch w=1u l=180n
M2844 t1033 nw294 0 0 nch w=1u l=180n
M2845 nw390 t1032 vdd vdd pch w=2u l=180n
M2846 nw390 t1032 0 0 nch w=1u l=180n
Cnw390 nw390 0 2f
CT1034 t1034 0 0.1f
M2847 t1034 nw329 0 0 nch w=1u l=180n
M2848 t1034 nw295 0 0 nch w=1u l=180n
CT1035 t1035 0 0.1f
M2849 t1035 nw329 vdd vdd pch w=2u l=180n
M2850 t1034 nw295 t1035 vdd pch w=2u l=180n
M2851 nw391 t1034 vdd vdd pch w=2u l=180n
M2852 nw391 t1034 0 0 nch w=1u l=180n
Cnw391 nw391 0 2f
CT1036 t1036 0 0.1f
CT1037 t1037 0 0.1f
CT1038 t1038 0 0.1f
M2853 t1036 nw330 vdd vdd pch w=2u l=180n
M2854 t1036 nw296 vdd vdd pch w=2u l=180n
CT1039 t1039 0 0.1f
M2855 t1036 nw330 t1039 0 nch w=1u l=180n
M2856 t1039 nw296 0 0 nch w=1u l=180n
M2857 t1037 nw330 vdd vdd pch w=2u l=180n
M2858 t1037 t1036 vdd vdd pch w=2u l=180n
CT1040 t1040 0 0.1f
M2859 t1037 nw330 t1040 0 nch w=1u l=180n
M2860 t1040 t1036 0 0 nch w=1u l=180n
M2861 t1038 nw296 vdd vdd pch w=2u l=180n
M2862 t1038 t1036 vdd vdd pch w=2u l=180n
CT1041 t1041 0 0.1f
M2863 t1038 nw296 t1041 0 nch w=1u l=180n
M2864 t1041 t1036 0 0 nch w=1u l=180n
M2865 nw392 t1037 vdd vdd pch w=2u l=180n
M2866 nw392 t1038 vdd vdd pch w=2u l=180n
CT1042 t1042 0 0.1f
M2867 nw392 t1037 t1042 0 nch w=1u l=180n
M2868 t1042 t1038 0 0 nch w=1u l=180n
Cnw392 nw392 0 2f
M2869 nw393 nw331 vdd vdd pch w=2u l=180n
M2870 nw393 nw297 vdd vdd pch w=2u l=180n
CT1043 t1043 0 0.1f
M2871 nw393 nw331 t1043 0 nch w=1u l=180n
M2872 t1043 nw297 0 0 nch w=1u l=180n
Cnw393 nw393 0 2f
M2873 nw394 nw332 0 0 nch w=1u l=180n
M2874 nw394 nw298 0 0 nch w=1u l=180n
CT1044 t1044 0 0.1f
M2875 t1044 nw332 vdd vdd pch w=2u l=180n
M2876 nw394 nw298 t1044 vdd pch w=2u l=180n
Cnw394 nw394 0 2f
CT1045 t1045 0 0.1f
M2877 t1045 nw333 vdd vdd pch w=2u l=180n
M2878 t1045 nw299 vdd vdd pch w=2u l=180n
CT1046 t1046 0 0.1f
M2879 t1045 nw333 t1046 0 nch w=1u l=180n
M2880 t1046 nw299 0 0 nch w=1u l=180n
M2881 nw395 t1045 vdd vdd pch w=2u l=180n
M2882 nw395 t1045 0 0 nch w=1u l=180n
Cnw395 nw395 0 2f
CT1047 t1047 0 0.1f
M2883 t1047 nw334 0 0 nch w=1u l=180n
M2884 t1047 nw300 0 0 nch w=1u l=180n
CT1048 t1048 0 0.1f
M2885 t1048 nw334 vdd vdd pch w=2u l=180n
M2886 t1047 nw300 t1048 vdd pch w=2u l=180n
M2887 nw396 t1047 vdd vdd pch w=2u l=180n
M2888 nw396 t1047 0 0 nch w=1u l=180n
Cnw396 nw396 0 2f
CT1049 t1049 0 0.1f
CT1050 t1050 0 0.1f
CT1051 t1051 0 0.1f
M2889 t1049 nw335 vdd vdd pch w=2u l=180n
M2890 t1049 nw301 vdd vdd pch w=2u l=180n
CT1052 t1052 0 0.1f
M2891 t1049 nw335 t1052 0 nch w=1u l=180n
M2892 t1052 nw301 0 0 nch w=1u l=180n
M2893 t1050 nw335 vdd vdd pch w=2u l=180n
M2894 t1050 t1049 vdd vdd pch w=2u l=180n
CT1053 t1053 0 0.1f
M2895 t1050 nw335 t1053 0 nch w=1u l=180n
M2896 t1053 t1049 0 0 nch w=1u l=180n
M2897 t1051 nw301 vdd vdd pch w=2u l=180n
M2898 t1051 t1049 vdd vdd pch w=2u l=180n
CT1054 t1054 0 0.1f
M2899 t1051 nw301 t1054 0 nch w=1u l=180n
M2900 t1054 t1049 0 0 nch w=1u l=180n
M2901 nw397 t1050 vdd vdd pch w=2u l=180n
M2902 nw397 t1051 vdd vdd pch w=2u l=180n
CT1055 t1055 0 0.1f
M2903 nw397 t1050 t1055 0 nch w=1u l=180n
M2904 t1055 t1051 0 0 nch w=1u l=180n
Cnw397 nw397 0 2f
M2905 nw398 nw336 vdd vdd pch w=2u l=180n
M2906 nw398 nw302 vdd vdd pch w=2u l=180n
CT1056 t1056 0 0.1f
M2907 nw398 nw336 t1056 0 nch w=1u l=180n
M2908 t1056 nw302 0 0 nch w=1u l=180n
Cnw398 nw398 0 2f
M2909 nw399 nw337 0 0 nch w=1u l=180n
M2910 nw399 nw303 0 0 nch w=1u l=180n
CT1057 t1057 0 0.1f
M2911 t1057 nw337 vdd vdd pch w=2u l=180n
M2912 nw399 nw303 t1057 vdd pch w=2u l=180n
Cnw399 nw399 0 2f
CT1058 t1058 0 0.1f
M2913 t1058 nw338 vdd vdd pch w=2u l=180n
M2914 t1058 nw304 vdd vdd pch w=2u l=180n
CT1059 t1059 0 0.1f
M2915 t1058 nw338 t1059 0 nch w=1u l=180n
M2916 t1059 nw304 0 0 nch w=1u l=180n
M2917 nw400 t1058 vdd vdd pch w=2u l=180n
M2918 nw400 t1058 0 0 nch w=1u l=180n
Cnw400 nw400 0 2f
CT1060 t1060 0 0.1f
M2919 t1060 nw339 0 0 nch w=1u l=180n
M2920 t1060 nw305 0 0 nch w=1u l=180n
CT1061 t1061 0 0.1f
M2921 t1061 nw339 vdd vdd pch w=2u l=180n
M2922 t1060 nw305 t1061 vdd pch w=2u l=180n
M2923 nw401 t1060 vdd vdd pch w=2u l=180n
M2924 nw401 t1060 0 0 nch w=1u l=180n
Cnw401 nw401 0 2f
CT1062 t1062 0 0.1f
CT1063 t1063 0 0.1f
CT1064 t1064 0 0.1f
M2925 t1062 nw340 vdd vdd pch w=2u l=180n
M2926 t1062 nw306 vdd vdd pch w=2u l=180n
CT1065 t1065 0 0.1f
M2927 t1062 nw340 t1065 0 nch w=1u l=180n
M2928 t1065 nw306 0 0 nch w=1u l=180n
M2929 t1063 nw340 vdd vdd pch w=2u l=180n
M2930 t1063 t1062 vdd vdd pch w=2u l=180n
CT1066 t1066 0 0.1f
M2931 t1063 nw340 t1066 0 nch w=1u l=180n
M2932 t1066 t1062 0 0 nch w=1u l=180n
M2933 t1064 nw306 vdd vdd pch w=2u l=180n
M2934 t1064 t1062 vdd vdd pch w=2u l=180n
CT1067 t1067 0 0.1f
M2935 t1064 nw306 t1067 0 nch w=1u l=180n
M2936 t1067 t1062 0 0 nch w=1u l=180n
M2937 nw402 t1063 vdd vdd pch w=2u l=180n
M2938 nw402 t1064 vdd vdd pch w=2u l=180n
CT1068 t1068 0 0.1f
M2939 nw402 t1063 t1068 0 nch w=1u l=180n
M2940 t1068 t1064 0 0 nch w=1u l=180n
Cnw402 nw402 0 2f
M2941 nw403 nw341 vdd vdd pch w=2u l=180n
M2942 nw403 nw307 vdd vdd pch w=2u l=180n
CT1069 t1069 0 0.1f
M2943 nw403 nw341 t1069 0 nch w=1u l=180n
M2944 t1069 nw307 0 0 nch w=1u l=180n
Cnw403 nw403 0 2f
M2945 nw404 nw342 0 0 nch w=1u l=180n
M2946 nw404 nw308 0 0 nch w=1u l=180n
CT1070 t1070 0 0.1f
M2947 t1070 nw342 vdd vdd pch w=2u l=180n
M2948 nw404 nw308 t1070 vdd pch w=2u l=180n
Cnw404 nw404 0 2f
CT1071 t1071 0 0.1f
M2949 t1071 nw343 vdd vdd pch w=2u l=180n
M2950 t1071 nw309 vdd vdd pch w=2u l=180n
CT1072 t1072 0 0.1f
M2951 t1071 nw343 t1072 0 nch w=1u l=180n
M2952 t1072 nw309 0 0 nch w=1u l=180n
M2953 nw405 t1071 vdd vdd pch w=2u l=180n
M2954 nw405 t1071 0 0 nch w=1u l=180n
Cnw405 nw405 0 2f
CT1073 t1073 0 0.1f
M2955 t1073 nw344 0 0 nch w=1u l=180n
M2956 t1073 nw310 0 0 nch w=1u l=180n
CT1074 t1074 0 0.1f
M2957 t1074 nw344 vdd vdd pch w=2u l=180n
M2958 t1073 nw310 t1074 vdd pch w=2u l=180n
M2959 nw406 t1073 vdd vdd pch w=2u l=180n
M2960 nw406 t1073 0 0 nch w=1u l=180n
Cnw406 nw406 0 2f
CT1075 t1075 0 0.1f
CT1076 t1076 0 0.1f
CT1077 t1077 0 0.1f
M2961 t1075 nw345 vdd vdd pch w=2u l=180n
M2962 t1075 nw311 vdd vdd pch w=2u l=180n
CT1078 t1078 0 0.1f
M2963 t1075 nw345 t1078 0 nch w=1u l=180n
M2964 t1078 nw311 0 0 nch w=1u l=180n
M2965 t1076 nw345 vdd vdd pch w=2u l=180n
M2966 t1076 t1075 vdd vdd pch w=2u l=180n
CT1079 t1079 0 0.1f
M2967 t1076 nw345 t1079 0 nch w=1u l=180n
M2968 t1079 t1075 0 0 nch w=1u l=180n
M2969 t1077 nw311 vdd vdd pch w=2u l=180n
M2970 t1077 t1075 vdd vdd pch w=2u l=180n
CT1080 t1080 0 0.1f
M2971 t1077 nw311 t1080 0 nch w=1u l=180n
M2972 t1080 t1075 0 0 nch w=1u l=180n
M2973 nw407 t1076 vdd vdd pch w=2u l=180n
M2974 nw407 t1077 vdd vdd pch w=2u l=180n
CT1081 t1081 0 0.1f
M2975 nw407 t1076 t1081 0 nch w=1u l=180n
M2976 t1081 t1077 0 0 nch w=1u l=180n
Cnw407 nw407 0 2f
M2977 nw408 nw346 vdd vdd pch w=2u l=180n
M2978 nw408 nw312 vdd vdd pch w=2u l=180n
CT1082 t1082 0 0.1f
M2979 nw408 nw346 t1082 0 nch w=1u l=180n
M2980 t1082 nw312 0 0 nch w=1u l=180n
Cnw408 nw408 0 2f
M2981 nw409 nw347 0 0 nch w=1u l=180n
M2982 nw409 nw313 0 0 nch w=1u l=180n
CT1083 t1083 0 0.1f
M2983 t1083 nw347 vdd vdd pch w=2u l=180n
M2984 nw409 nw313 t1083 vdd pch w=2u l=180n
Cnw409 nw409 0 2f
CT1084 t1084 0 0.1f
M2985 t1084 nw348 vdd vdd pch w=2u l=180n
M2986 t1084 nw314 vdd vdd pch w=2u l=180n
CT1085 t1085 0 0.1f
M2987 t1084 nw348 t1085 0 nch w=1u l=180n
M2988 t1085 nw314 0 0 nch w=1u l=180n
M2989 nw410 t1084 vdd vdd pch w=2u l=180n
M2990 nw410 t1084 0 0 nch w=1u l=180n
Cnw410 nw410 0 2f
CT1086 t1086 0 0.1f
M2991 t1086 nw349 0 0 nch w=1u l=180n
M2992 t1086 nw315 0 0 nch w=1u l=180n
CT1087 t1087 0 0.1f
M2993 t1087 nw349 vdd vdd pch w=2u l=180n
M2994 t1086 nw315 t1087 vdd pch w=2u l=180n
M2995 nw411 t1086 vdd vdd pch w=2u l=180n
M2996 nw411 t1086 0 0 nch w=1u l=180n
Cnw411 nw411 0 2f
CT1088 t1088 0 0.1f
CT1089 t1089 0 0.1f
CT1090 t1090 0 0.1f
M2997 t1088 nw350 vdd vdd pch w=2u l=180n
M2998 t1088 nw316 vdd vdd pch w=2u l=180n
CT1091 t1091 0 0.1f
M2999 t1088 nw350 t1091 0 nch w=1u l=180n
M3000 t1091 nw316 0 0 nch w=1u l=180n
M3001 t1089 nw350 vdd vdd pch w=2u l=180n
M3002 t1089 t1088 vdd vdd pch w=2u l=180n
CT1092 t1092 0 0.1f
M3003 t1089 nw350 t1092 0 nch w=1u l=180n
M3004 t1092 t1088 0 0 nch w=1u l=180n
M3005 t1090 nw316 vdd vdd pch w=2u l=180n
M3006 t1090 t1088 vdd vdd pch w=2u l=180n
CT1093 t1093 0 0.1f
M3007 t1090 nw316 t1093 0 nch w=1u l=180n
M3008 t1093 t1088 0 0 nch w=1u l=180n
M3009 nw412 t1089 vdd vdd pch w=2u l=180n
M3010 nw412 t1090 vdd vdd pch w=2u l=180n
CT1094 t1094 0 0.1f
M3011 nw412 t1089 t1094 0 nch w=1u l=180n
M3012 t1094 t1090 0 0 nch w=1u l=180n
Cnw412 nw412 0 2f
M3013 nw413 nw351 vdd vdd pch w=2u l=180n
M3014 nw413 nw317 vdd vdd pch w=2u l=180n
CT1095 t1095 0 0.1f
M3015 nw413 nw351 t1095 0 nch w=1u l=180n
M3016 t1095 nw317 0 0 nch w=1u l=180n
Cnw413 nw413 0 2f
M3017 nw414 nw352 0 0 nch w=1u l=180n
M3018 nw414 nw318 0 0 nch w=1u l=180n
CT1096 t1096 0 0.1f
M3019 t1096 nw352 vdd vdd pch w=2u l=180n
M3020 nw414 nw318 t1096 vdd pch w=2u l=180n
Cnw414 nw414 0 2f
CT1097 t1097 0 0.1f
M3021 t1097 nw353 vdd vdd pch w=2u l=180n
M3022 t1097 nw319 vdd vdd pch w=2u l=180n
CT1098 t1098 0 0.1f
M3023 t1097 nw353 t1098 0 nch w=1u l=180n
M3024 t1098 nw319 0 0 nch w=1u l=180n
M3025 nw415 t1097 vdd vdd pch w=2u l=180n
M3026 nw415 t1097 0 0 nch w=1u l=180n
Cnw415 nw415 0 2f
CT1099 t1099 0 0.1f
M3027 t1099 nw354 0 0 nch w=1u l=180n
M3028 t1099 nw320 0 0 nch w=1u l=180n
CT1100 t1100 0 0.1f
M3029 t1100 nw354 vdd vdd pch w=2u l=180n
M3030 t1099 nw320 t1100 vdd pch w=2u l=180n
M3031 nw416 t1099 vdd vdd pch w=2u l=180n
M3032 nw416 t1099 0 0 nch w=1u l=180n
Cnw416 nw416 0 2f
CT1101 t1101 0 0.1f
CT1102 t1102 0 0.1f
CT1103 t1103 0 0.1f
M3033 t1101 nw355 vdd vdd pch w=2u l=180n
M3034 t1101 nw321 vdd vdd pch w=2u l=180n
CT1104 t1104 0 0.1f
M3035 t1101 nw355 t1104 0 nch w=1u l=180n
M3036 t1104 nw321 0 0 nch w=1u l=180n
M3037 t1102 nw355 vdd vdd pch w=2u l=180n
M3038 t1102 t1101 vdd vdd pch w=2u l=180n
CT1105 t1105 0 0.1f
M3039 t1102 nw355 t1105 0 nch w=1u l=180n
M3040 t1105 t1101 0 0 nch w=1u l=180n
M3041 t1103 nw321 vdd vdd pch w=2u l=180n
M3042 t1103 t1101 vdd vdd pch w=2u l=180n
CT1106 t1106 0 0.1f
M3043 t1103 nw321 t1106 0 nch w=1u l=180n
M3044 t1106 t1101 0 0 nch w=1u l=180n
M3045 nw417 t1102 vdd vdd pch w=2u l=180n
M3046 nw417 t1103 vdd vdd pch w=2u l=180n
CT1107 t1107 0 0.1f
M3047 nw417 t1102 t1107 0 nch w=1u l=180n
M3048 t1107 t1103 0 0 nch w=1u l=180n
Cnw417 nw417 0 2f
M3049 nw418 nw356 vdd vdd pch w=2u l=180n
M3050 nw418 nw322 vdd vdd pch w=2u l=180n
CT1108 t1108 0 0.1f
M3051 nw418 nw356 t1108 0 nch w=1u l=180n
M3052 t1108 nw322 0 0 nch w=1u l=180n
Cnw418 nw418 0 2f
M3053 nw419 nw357 0 0 nch w=1u l=180n
M3054 nw419 nw323 0 0 nch w=1u l=180n
CT1109 t1109 0 0.1f
M3055 t1109 nw357 vdd vdd pch w=2u l=180n
M3056 nw419 nw323 t1109 vdd pch w=2u l=180n
Cnw419 nw419 0 2f
CT1110 t1110 0 0.1f
M3057 t1110 nw358 vdd vdd pch w=2u l=180n
M3058 t1110 nw324 vdd vdd pch w=2u l=180n
CT1111 t1111 0 0.1f
M3059 t1110 nw358 t1111 0 nch w=1u l=180n
M3060 t1111 nw324 0 0 nch w=1u l=180n
M3061 nw420 t1110 vdd vdd pch w=2u l=180n
M3062 nw420 t1110 0 0 nch w=1u l=180n
Cnw420 nw420 0 2f
CT1112 t1112 0 0.1f
M3063 t1112 nw359 0 0 nch w=1u l=180n
M3064 t1112 nw325 0 0 nch w=1u l=180n
CT1113 t1113 0 0.1f
M3065 t1113 nw359 vdd vdd pch w=2u l=180n
M3066 t1112 nw325 t1113 vdd pch w=2u l=180n
M3067 nw421 t1112 vdd vdd pch w=2u l=180n
M3068 nw421 t1112 0 0 nch w=1u l=180n
Cnw421 nw421 0 2f
CT1114 t1114 0 0.1f
CT1115 t1115 0 0.1f
CT1116 t1116 0 0.1f
M3069 t1114 nw360 vdd vdd pch w=2u l=180n
M3070 t1114 nw326 vdd vdd pch w=2u l=180n
CT1117 t1117 0 0.1f
M3071 t1114 nw360 t1117 0 nch w=1u l=180n
M3072 t1117 nw326 0 0 nch w=1u l=180n
M3073 t1115 nw360 vdd vdd pch w=2u l=180n
M3074 t1115 t1114 vdd vdd pch w=2u l=180n
CT1118 t1118 0 0.1f
M3075 t1115 nw360 t1118 0 nch w=1u l=180n
M3076 t1118 t1114 0 0 nch w=1u l=180n
M3077 t1116 nw326 vdd vdd pch w=2u l=180n
M3078 t1116 t1114 vdd vdd pch w=2u l=180n
CT1119 t1119 0 0.1f
M3079 t1116 nw326 t1119 0 nch w=1u l=180n
M3080 t1119 t1114 0 0 nch w=1u l=180n
M3081 nw422 t1115 vdd vdd pch w=2u l=180n
M3082 nw422 t1116 vdd vdd pch w=2u l=180n
CT1120 t1120 0 0.1f
M3083 nw422 t1115 t1120 0 nch w=1u l=180n
M3084 t1120 t1116 0 0 nch w=1u l=180n
Cnw422 nw422 0 2f
M3085 nw423 nw361 vdd vdd pch w=2u l=180n
M3086 nw423 nw327 vdd vdd pch w=2u l=180n
CT1121 t1121 0 0.1f
M3087 nw423 nw361 t1121 0 nch w=1u l=180n
M3088 t1121 nw327 0 0 nch w=1u l=180n
Cnw423 nw423 0 2f
M3089 nw424 nw362 0 0 nch w=1u l=180n
M3090 nw424 nw328 0 0 nch w=1u l=180n
CT1122 t1122 0 0.1f
M3091 t1122 nw362 vdd vdd pch w=2u l=180n
M3092 nw424 nw328 t1122 vdd pch w=2u l=180n
Cnw424 nw424 0 2f
CT1123 t1123 0 0.1f
M3093 t1123 nw363 vdd vdd pch w=2u l=180n
M3094 t1123 nw329 vdd vdd pch w=2u l=180n
CT1124 t1124 0 0.1f
M3095 t1123 nw363 t1124 0 nch w=1u l=180n
M3096 t1124 nw329 0 0 nch w=1u l=180n
M3097 nw425 t1123 vdd vdd pch w=2u l=180n
M3098 nw425 t1123 0 0 nch w=1u l=180n
Cnw425 nw425 0 2f
CT1125 t1125 0 0.1f
M3099 t1125 nw364 0 0 nch w=1u l=180n
M3100 t1125 nw330 0 0 nch w=1u l=180n
CT1126 t1126 0 0.1f
M3101 t1126 nw364 vdd vdd pch w=2u l=180n
M3102 t1125 nw330 t1126 vdd pch w=2u l=180n
M3103 nw426 t1125 vdd vdd pch w=2u l=180n
M3104 nw426 t1125 0 0 nch w=1u l=180n
Cnw426 nw426 0 2f
CT1127 t1127 0 0.1f
CT1128 t1128 0 0.1f
CT1129 t1129 0 0.1f
M3105 t1127 nw365 vdd vdd pch w=2u l=180n
M3106 t1127 nw331 vdd vdd pch w=2u l=180n
CT1130 t1130 0 0.1f
M3107 t1127 nw365 t1130 0 nch w=1u l=180n
M3108 t1130 nw331 0 0 nch w=1u l=180n
M3109 t1128 nw365 vdd vdd pch w=2u l=180n
M3110 t1128 t1127 vdd vdd pch w=2u l=180n
CT1131 t1131 0 0.1f
M3111 t1128 nw365 t1131 0 nch w=1u l=180n
M3112 t1131 t1127 0 0 nch w=1u l=180n
M3113 t1129 nw331 vdd vdd pch w=2u l=180n
M3114 t1129 t1127 vdd vdd pch w=2u l=180n
CT1132 t1132 0 0.1f
M3115 t1129 nw331 t1132 0 nch w=1u l=180n
M3116 t1132 t1127 0 0 nch w=1u l=180n
M3117 nw427 t1128 vdd vdd pch w=2u l=180n
M3118 nw427 t1129 vdd vdd pch w=2u l=180n
CT1133 t1133 0 0.1f
M3119 nw427 t1128 t1133 0 nch w=1u l=180n
M3120 t1133 t1129 0 0 nch w=1u l=180n
Cnw427 nw427 0 2f
M3121 nw428 nw366 vdd vdd pch w=2u l=180n
M3122 nw428 nw332 vdd vdd pch w=2u l=180n
CT1134 t1134 0 0.1f
M3123 nw428 nw366 t1134 0 nch w=1u l=180n
M3124 t1134 nw332 0 0 nch w=1u l=180n
Cnw428 nw428 0 2f
M3125 nw429 nw367 0 0 nch w=1u l=180n
M3126 nw429 nw333 0 0 nch w=1u l=180n
CT1135 t1135 0 0.1f
M3127 t1135 nw367 vdd vdd pch w=2u l=180n
M3128 nw429 nw333 t1135 vdd pch w=2u l=180n
Cnw429 nw429 0 2f
CT1136 t1136 0 0.1f
M3129 t1136 nw368 vdd vdd pch w=2u l=180n
M3130 t1136 nw334 vdd vdd pch w=2u l=180n
CT1137 t1137 0 0.1f
M3131 t1136 nw368 t1137 0 nch w=1u l=180n
M3132 t1137 nw334 0 0 nch w=1u l=180n
M3133 nw430 t1136 vdd vdd pch w=2u l=180n
M3134 nw430 t1136 0 0 nch w=1u l=180n
Cnw430 nw430 0 2f
CT1138 t1138 0 0.1f
M3135 t1138 nw369 0 0 nch w=1u l=180n
M3136 t1138 nw335 0 0 nch w=1u l=180n
CT1139 t1139 0 0.1f
M3137 t1139 nw369 vdd vdd pch w=2u l=180n
M3138 t1138 nw335 t1139 vdd pch w=2u l=180n
M3139 nw431 t1138 vdd vdd pch w=2u l=180n
M3140 nw431 t1138 0 0 nch w=1u l=180n
Cnw431 nw431 0 2f
CT1140 t1140 0 0.1f
CT1141 t1141 0 0.1f
CT1142 t1142 0 0.1f
M3141 t1140 nw370 vdd vdd pch w=2u l=180n
M3142 t1140 nw336 vdd vdd pch w=2u l=180n
CT1143 t1143 0 0.1f
M3143 t1140 nw370 t1143 0 nch w=1u l=180n
M3144 t1143 nw336 0 0 nch w=1u l=180n
M3145 t1141 nw370 vdd vdd pch w=2u l=180n
M3146 t1141 t1140 vdd vdd pch w=2u l=180n
CT1144 t1144 0 0.1f
M3147 t1141 nw370 t1144 0 nch w=1u l=180n
M3148 t1144 t1140 0 0 nch w=1u l=180n
M3149 t1142 nw336 vdd vdd pch w=2u l=180n
M3150 t1142 t1140 vdd vdd pch w=2u l=180n
CT1145 t1145 0 0.1f
M3151 t1142 nw336 t1145 0 nch w=1u l=180n
M3152 t1145 t1140 0 0 nch w=1u l=180n
M3153 nw432 t1141 vdd vdd pch w=2u l=180n
M3154 nw432 t1142 vdd vdd pch w=2u l=180n
CT1146 t1146 0 0.1f
M3155 nw432 t1141 t1146 0 nch w=1u l=180n
M3156 t1146 t1142 0 0 nch w=1u l=180n
Cnw432 nw432 0 2f
M3157 nw433 nw371 vdd vdd pch w=2u l=180n
M3158 nw433 nw337 vdd vdd pch w=2u l=180n
CT1147 t1147 0 0.1f
M3159 nw433 nw371 t1147 0 nch w=1u l=180n
M3160 t1147 nw337 0 0 nch w=1u l=180n
Cnw433 nw433 0 2f
M3161 nw434 nw372 0 0 nch w=1u l=180n
M3162 nw434 nw338 0 0 nch w=1u l=180n
CT1148 t1148 0 0.1f
M3163 t1148 nw372 vdd vdd pch w=2u l=180n
M3164 nw434 nw338 t1148 vdd pch w=2u l=180n
Cnw434 nw434 0 2f
CT1149 t1149 0 0.1f
M3165 t1149 nw373 vdd vdd pch w=2u l=180n
M3166 t1149 nw339 vdd vdd pch w=2u l=180n
CT1150 t1150 0 0.1f
M3167 t1149 nw373 t1150 0 nch w=1u l=180n
M3168 t1150 nw339 0 0 nch w=1u l=180n
M3169 nw435 t1149 vdd vdd pch w=2u l=180n
M3170 nw435 t1149 0 0 nch w=1u l=180n
Cnw435 nw435 0 2f
CT1151 t1151 0 0.1f
M3171 t1151 nw374 0 0 nch w=1u l=180n
M3172 t1151 nw340 0 0 nch w=1u l=180n
CT1152 t1152 0 0.1f
M3173 t1152 nw374 vdd vdd pch w=2u l=180n
M3174 t1151 nw340 t1152 vdd pch w=2u l=180n
M3175 nw436 t1151 vdd vdd pch w=2u l=180n
M3176 nw436 t1151 0 0 nch w=1u l=180n
Cnw436 nw436 0 2f
CT1153 t1153 0 0.1f
CT1154 t1154 0 0.1f
CT1155 t1155 0 0.1f
M3177 t1153 nw375 vdd vdd pch w=2u l=180n
M3178 t1153 nw341 vdd vdd pch w=2u l=180n
CT1156 t1156 0 0.1f
M3179 t1153 nw375 t1156 0 nch w=1u l=180n
M3180 t1156 nw341 0 0 nch w=1u l=180n
M3181 t1154 nw375 vdd vdd pch w=2u l=180n
M3182 t1154 t1153 vdd vdd pch w=2u l=180n
CT1157 t1157 0 0.1f
M3183 t1154 nw375 t1157 0 nch w=1u l=180n
M3184 t1157 t1153 0 0 nch w=1u l=180n
M3185 t1155 nw341 vdd vdd pch w=2u l=180n
M3186 t1155 t1153 vdd vdd pch w=2u l=180n
CT1158 t1158 0 0.1f
M3187 t1155 nw341 t1158 0 nch w=1u l=180n
M3188 t1158 t1153 0 0 nch w=1u l=180n
M3189 nw437 t1154 vdd vdd pch w=2u l=180n
M3190 nw437 t1155 vdd vdd pch w=2u l=180n
CT1159 t1159 0 0.1f
M3191 nw437 t1154 t1159 0 nch w=1u l=180n
M3192 t1159 t1155 0 0 nch w=1u l=180n
Cnw437 nw437 0 2f
M3193 nw438 nw376 vdd vdd pch w=2u l=180n
M3194 nw438 nw342 vdd vdd pch w=2u l=180n
CT1160 t1160 0 0.1f
M3195 nw438 nw376 t1160 0 nch w=1u l=180n
M3196 t1160 nw342 0 0 nch w=1u l=180n
Cnw438 nw438 0 2f
M3197 nw439 nw377 0 0 nch w=1u l=180n
M3198 nw439 nw343 0 0 nch w=1u l=180n
CT1161 t1161 0 0.1f
M3199 t1161 nw377 vdd vdd pch w=2u l=180n
M3200 nw439 nw343 t1161 vdd pch w=2u l=180n
Cnw439 nw439 0 2f
CT1162 t1162 0 0.1f
M3201 t1162 nw378 vdd vdd pch w=2u l=180n
M3202 t1162 nw344 vdd vdd pch w=2u l=180n
CT1163 t1163 0 0.1f
M3203 t1162 nw378 t1163 0 nch w=1u l=180n
M3204 t1163 nw344 0 0 nch w=1u l=180n
M3205 nw440 t1162 vdd vdd pch w=2u l=180n
M3206 nw440 t1162 0 0 nch w=1u l=180n
Cnw440 nw440 0 2f
CT1164 t1164 0 0.1f
M3207 t1164 nw379 0 0 nch w=1u l=180n
M3208 t1164 nw345 0 0 nch w=1u l=180n
CT1165 t1165 0 0.1f
M3209 t1165 nw379 vdd vdd pch w=2u l=180n
M3210 t1164 nw345 t1165 vdd pch w=2u l=180n
M3211 nw441 t1164 vdd vdd pch w=2u l=180n
M3212 nw441 t1164 0 0 nch w=1u l=180n
Cnw441 nw441 0 2f
CT1166 t1166 0 0.1f
CT1167 t1167 0 0.1f
CT1168 t1168 0 0.1f
M3213 t1166 nw380 vdd vdd pch w=2u l=180n
M3214 t1166 nw346 vdd vdd pch w=2u l=180n
CT1169 t1169 0 0.1f
M3215 t1166 nw380 t1169 0 nch w=1u l=180n
M3216 t1169 nw346 0 0 nch w=1u l=180n
M3217 t1167 nw380 vdd vdd pch w=2u l=180n
M3218 t1167 t1166 vdd vdd pch w=2u l=180n
CT1170 t1170 0 0.1f
M3219 t1167 nw380 t1170 0 nch w=1u l=180n
M3220 t1170 t1166 0 0 nch w=1u l=180n
M3221 t1168 nw346 vdd vdd pch w=2u l=180n
M3222 t1168 t1166 vdd vdd pch w=2u l=180n
CT1171 t1171 0 0.1f
M3223 t1168 nw346 t1171 0 nch w=1u l=180n
M3224 t1171 t1166 0 0 nch w=1u l=180n
M3225 nw442 t1167 vdd vdd pch w=2u l=180n
M3226 nw442 t1168 vdd vdd pch w=2u l=180n
CT1172 t1172 0 0.1f
M3227 nw442 t1167 t1172 0 nch w=1u l=180n
M3228 t1172 t1168 0 0 nch w=1u l=180n
Cnw442 nw442 0 2f
M3229 nw443 nw381 vdd vdd pch w=2u l=180n
M3230 nw443 nw347 vdd vdd pch w=2u l=180n
CT1173 t1173 0 0.1f
M3231 nw443 nw381 t1173 0 nch w=1u l=180n
M3232 t1173 nw347 0 0 nch w=1u l=180n
Cnw443 nw443 0 2f
M3233 nw444 nw382 0 0 nch w=1u l=180n
M3234 nw444 nw348 0 0 nch w=1u l=180n
CT1174 t1174 0 0.1f
M3235 t1174 nw382 vdd vdd pch w=2u l=180n
M3236 nw444 nw348 t1174 vdd pch w=2u l=180n
Cnw444 nw444 0 2f
CT1175 t1175 0 0.1f
M3237 t1175 nw383 vdd vdd pch w=2u l=180n
M3238 t1175 nw349 vdd vdd pch w=2u l=180n
CT1176 t1176 0 0.1f
M3239 t1175 nw383 t1176 0 nch w=1u l=180n
M3240 t1176 nw349 0 0 nch w=1u l=180n
M3241 nw445 t1175 vdd vdd pch w=2u l=180n
M3242 nw445 t1175 0 0 nch w=1u l=180n
Cnw445 nw445 0 2f
CT1177 t1177 0 0.1f
M3243 t1177 nw384 0 0 nch w=1u l=180n
M3244 t1177 nw350 0 0 nch w=1u l=180n
CT1178 t1178 0 0.1f
M3245 t1178 nw384 vdd vdd pch w=2u l=180n
M3246 t1177 nw350 t1178 vdd pch w=2u l=180n
M3247 nw446 t1177 vdd vdd pch w=2u l=180n
M3248 nw446 t1177 0 0 nch w=1u l=180n
Cnw446 nw446 0 2f
CT1179 t1179 0 0.1f
CT1180 t1180 0 0.1f
CT1181 t1181 0 0.1f
M3249 t1179 nw385 vdd vdd pch w=2u l=180n
M3250 t1179 nw351 vdd vdd pch w=2u l=180n
CT1182 t1182 0 0.1f
M3251 t1179 nw385 t1182 0 nch w=1u l=180n
M3252 t1182 nw351 0 0 nch w=1u l=180n
M3253 t1180 nw385 vdd vdd pch w=2u l=180n
M3254 t1180 t1179 vdd vdd pch w=2u l=180n
CT1183 t1183 0 0.1f
M3255 t1180 nw385 t1183 0 nch w=1u l=180n
M3256 t1183 t1179 0 0 nch w=1u l=180n
M3257 t1181 nw351 vdd vdd pch w=2u l=180n
M3258 t1181 t1179 vdd vdd pch w=2u l=180n
CT1184 t1184 0 0.1f
M3259 t1181 nw351 t1184 0 nch w=1u l=180n
M3260 t1184 t1179 0 0 nch w=1u l=180n
M3261 nw447 t1180 vdd vdd pch w=2u l=180n
M3262 nw447 t1181 vdd vdd pch w=2u l=180n
CT1185 t1185 0 0.1f
M3263 nw447 t1180 t1185 0 nch w=1u l=180n
M3264 t1185 t1181 0 0 nch w=1u l=180n
Cnw447 nw447 0 2f
M3265 nw448 nw386 vdd vdd pch w=2u l=180n
M3266 nw448 nw352 vdd vdd pch w=2u l=180n
CT1186 t1186 0 0.1f
M3267 nw448 nw386 t1186 0 nch w=1u l=180n
M3268 t1186 nw352 0 0 nch w=1u l=180n
Cnw448 nw448 0 2f
M3269 nw449 nw387 0 0 nch w=1u l=180n
M3270 nw449 nw353 0 0 nch w=1u l=180n
CT1187 t1187 0 0.1f
M3271 t1187 nw387 vdd vdd pch w=2u l=180n
M3272 nw449 nw353 t1187 vdd pch w=2u l=180n
Cnw449 nw449 0 2f
CT1188 t1188 0 0.1f
M3273 t1188 nw388 vdd vdd pch w=2u l=180n
M3274 t1188 nw354 vdd vdd pch w=2u l=180n
CT1189 t1189 0 0.1f
M3275 t1188 nw388 t1189 0 nch w=1u l=180n
M3276 t1189 nw354 0 0 nch w=1u l=180n
M3277 nw450 t1188 vdd vdd pch w=2u l=180n
M3278 nw450 t1188 0 0 nch w=1u l=180n
Cnw450 nw450 0 2f
CT1190 t1190 0 0.1f
M3279 t1190 nw389 0 0 nch w=1u l=180n
M3280 t1190 nw355 0 0 nch w=1u l=180n
CT1191 t1191 0 0.1f
M3281 t1191 nw389 vdd vdd pch w=2u l=180n
M3282 t1190 nw355 t1191 vdd pch w=2u l=180n
M3283 nw451 t1190 vdd vdd pch w=2u l=180n
M3284 nw451 t1190 0 0 nch w=1u l=180n
Cnw451 nw451 0 2f
CT1192 t1192 0 0.1f
CT1193 t1193 0 0.1f
CT1194 t1194 0 0.1f
M3285 t1192 nw390 vdd vdd pch w=2u l=180n
M3286 t1192 nw356 vdd vdd pch w=2u l=180n
CT1195 t1195 0 0.1f
M3287 t1192 nw390 t1195 0 nch w=1u l=180n
M3288 t1195 nw356 0 0 nch w=1u l=180n
M3289 t1193 nw390 vdd vdd pch w=2u l=180n
M3290 t1193 t1192 vdd vdd pch w=2u l=180n
CT1196 t1196 0 0.1f
M3291 t1193 nw390 t1196 0 nch w=1u l=180n
M3292 t1196 t1192 0 0 nch w=1u l=180n
M3293 t1194 nw356 vdd vdd pch w=2u l=180n
M3294 t1194 t1192 vdd vdd pch w=2u l=180n
CT1197 t1197 0 0.1f
M3295 t1194 nw356 t1197 0 nch w=1u l=180n
M3296 t1197 t1192 0 0 nch w=1u l=180n
M3297 nw452 t1193 vdd vdd pch w=2u l=180n
M3298 nw452 t1194 vdd vdd pch w=2u l=180n
CT1198 t1198 0 0.1f
M3299 nw452 t1193 t1198 0 nch w=1u l=180n
M3300 t1198 t1194 0 0 nch w=1u l=180n
Cnw452 nw452 0 2f
M3301 nw453 nw391 vdd vdd pch w=2u l=180n
M3302 nw453 nw357 vdd vdd pch w=2u l=180n
CT1199 t1199 0 0.1f
M3303 nw453 nw391 t1199 0 nch w=1u l=180n
M3304 t1199 nw357 0 0 nch w=1u l=180n
Cnw453 nw453 0 2f
M3305 nw454 nw392 0 0 nch w=1u l=180n
M3306 nw454 nw358 0 0 nch w=1u l=180n
CT1200 t1200 0 0.1f
M3307 t1200 nw392 vdd vdd pch w=2u l=180n
M3308 nw454 nw358 t1200 vdd pch w=2u l=180n
Cnw454 nw454 0 2f
CT1201 t1201 0 0.1f
M3309 t1201 nw393 vdd vdd pch w=2u l=180n
M3310 t1201 nw359 vdd vdd pch w=2u l=180n
CT1202 t1202 0 0.1f
M3311 t1201 nw393 t1202 0 nch w=1u l=180n
M3312 t1202 nw359 0 0 nch w=1u l=180n
M3313 nw455 t1201 vdd vdd pch w=2u l=180n
M3314 nw455 t1201 0 0 nch w=1u l=180n
Cnw455 nw455 0 2f
CT1203 t1203 0 0.1f
M3315 t1203 nw394 0 0 nch w=1u l=180n
M3316 t1203 nw360 0 0 nch w=1u l=180n
CT1204 t1204 0 0.1f
M3317 t1204 nw394 vdd vdd pch w=2u l=180n
M3318 t1203 nw360 t1204 vdd pch w=2u l=180n
M3319 nw456 t1203 vdd vdd pch w=2u l=180n
M3320 nw456 t1203 0 0 nch w=1u l=180n
Cnw456 nw456 0 2f
CT1205 t1205 0 0.1f
CT1206 t1206 0 0.1f
CT1207 t1207 0 0.1f
M3321 t1205 nw395 vdd vdd pch w=2u l=180n
M3322 t1205 nw361 vdd vdd pch w=2u l=180n
CT1208 t1208 0 0.1f
M3323 t1205 nw395 t1208 0 nch w=1u l=180n
M3324 t1208 nw361 0 0 nch w=1u l=180n
M3325 t1206 nw395 vdd vdd pch w=2u l=180n
M3326 t1206 t1205 vdd vdd pch w=2u l=180n
CT1209 t1209 0 0.1f
M3327 t1206 nw395 t1209 0 nch w=1u l=180n
M3328 t1209 t1205 0 0 nch w=1u l=180n
M3329 t1207 nw361 vdd vdd pch w=2u l=180n
M3330 t1207 t1205 vdd vdd pch w=2u l=180n
CT1210 t1210 0 0.1f
M3331 t1207 nw361 t1210 0 nch w=1u l=180n
M3332 t1210 t1205 0 0 nch w=1u l=180n
M3333 nw457 t1206 vdd vdd pch w=2u l=180n
M3334 nw457 t1207 vdd vdd pch w=2u l=180n
CT1211 t1211 0 0.1f
M3335 nw457 t1206 t1211 0 nch w=1u l=180n
M3336 t1211 t1207 0 0 nch w=1u l=180n
Cnw457 nw457 0 2f
M3337 nw458 nw396 vdd vdd pch w=2u l=180n
M3338 nw458 nw362 vdd vdd pch w=2u l=180n
CT1212 t1212 0 0.1f
M3339 nw458 nw396 t1212 0 nch w=1u l=180n
M3340 t1212 nw362 0 0 nch w=1u l=180n
Cnw458 nw458 0 2f
M3341 nw459 nw397 0 0 nch w=1u l=180n
M3342 nw459 nw363 0 0 nch w=1u l=180n
CT1213 t1213 0 0.1f
M3343 t1213 nw397 vdd vdd pch w=2u l=180n
M3344 nw459 nw363 t1213 vdd pch w=2u l=180n
Cnw459 nw459 0 2f
CT1214 t1214 0 0.1f
M3345 t1214 nw398 vdd vdd pch w=2u l=180n
M3346 t1214 nw364 vdd vdd pch w=2u l=180n
CT1215 t1215 0 0.1f
M3347 t1214 nw398 t1215 0 nch w=1u l=180n
M3348 t1215 nw364 0 0 nch w=1u l=180n
M3349 nw460 t1214 vdd vdd pch w=2u l=180n
M3350 nw460 t1214 0 0 nch w=1u l=180n
Cnw460 nw460 0 2f
CT1216 t1216 0 0.1f
M3351 t1216 nw399 0 0 nch w=1u l=180n
M3352 t1216 nw365 0 0 nch w=1u l=180n
CT1217 t1217 0 0.1f
M3353 t1217 nw399 vdd vdd pch w=2u l=180n
M3354 t1216 nw365 t1217 vdd pch w=2u l=180n
M3355 nw461 t1216 vdd vdd pch w=2u l=180n
M3356 nw461 t1216 0 0 nch w=1u l=180n
Cnw461 nw461 0 2f
CT1218 t1218 0 0.1f
CT1219 t1219 0 0.1f
CT1220 t1220 0 0.1f
M3357 t1218 nw400 vdd vdd pch w=2u l=180n
M3358 t1218 nw366 vdd vdd pch w=2u l=180n
CT1221 t1221 0 0.1f
M3359 t1218 nw400 t1221 0 nch w=1u l=180n
M3360 t1221 nw366 0 0 nch w=1u l=180n
M3361 t1219 nw400 vdd vdd pch w=2u l=180n
M3362 t1219 t1218 vdd vdd pch w=2u l=180n
CT1222 t1222 0 0.1f
M3363 t1219 nw400 t1222 0 nch w=1u l=180n
M3364 t1222 t1218 0 0 nch w=1u l=180n
M3365 t1220 nw366 vdd vdd pch w=2u l=180n
M3366 t1220 t1218 vdd vdd pch w=2u l=180n
CT1223 t1223 0 0.1f
M3367 t1220 nw366 t1223 0 nch w=1u l=180n
M3368 t1223 t1218 0 0 nch w=1u l=180n
M3369 nw462 t1219 vdd vdd pch w=2u l=180n
M3370 nw462 t1220 vdd vdd pch w=2u l=180n
CT1224 t1224 0 0.1f
M3371 nw462 t1219 t1224 0 nch w=1u l=180n
M3372 t1224 t1220 0 0 nch w=1u l=180n
Cnw462 nw462 0 2f
M3373 nw463 nw401 vdd vdd pch w=2u l=180n
M3374 nw463 nw367 vdd vdd pch w=2u l=180n
CT1225 t1225 0 0.1f
M3375 nw463 nw401 t1225 0 nch w=1u l=180n
M3376 t1225 nw367 0 0 nch w=1u l=180n
Cnw463 nw463 0 2f
M3377 nw464 nw402 0 0 nch w=1u l=180n
M3378 nw464 nw368 0 0 nch w=1u l=180n
CT1226 t1226 0 0.1f
M3379 t1226 nw402 vdd vdd pch w=2u l=180n
M3380 nw464 nw368 t1226 vdd pch w=2u l=180n
Cnw464 nw464 0 2f
CT1227 t1227 0 0.1f
M3381 t1227 nw403 vdd vdd pch w=2u l=180n
M3382 t1227 nw369 vdd vdd pch w=2u l=180n
CT1228 t1228 0 0.1f
M3383 t1227 nw403 t1228 0 nch w=1u l=180n
M3384 t1228 nw369 0 0 nch w=1u l=180n
M3385 nw465 t1227 vdd vdd pch w=2u l=180n
M3386 nw465 t1227 0 0 nch w=1u l=180n
Cnw465 nw465 0 2f
CT1229 t1229 0 0.1f
M3387 t1229 nw404 0 0 nch w=1u l=180n
M3388 t1229 nw370 0 0 nch w=1u l=180n
CT1230 t1230 0 0.1f
M3389 t1230 nw404 vdd vdd pch w=2u l=180n
M3390 t1229 nw370 t1230 vdd pch w=2u l=180n
M3391 nw466 t1229 vdd vdd pch w=2u l=180n
M3392 nw466 t1229 0 0 nch w=1u l=180n
Cnw466 nw466 0 2f
CT1231 t1231 0 0.1f
CT1232 t1232 0 0.1f
CT1233 t1233 0 0.1f
M3393 t1231 nw405 vdd vdd pch w=2u l=180n
M3394 t1231 nw371 vdd vdd pch w=2u l=180n
CT1234 t1234 0 0.1f
M3395 t1231 nw405 t1234 0 nch w=1u l=180n
M3396 t1234 nw371 0 0 nch w=1u l=180n
M3397 t1232 nw405 vdd vdd pch w=2u l=180n
M3398 t1232 t1231 vdd vdd pch w=2u l=180n
CT1235 t1235 0 0.1f
M3399 t1232 nw405 t1235 0 nch w=1u l=180n
M3400 t1235 t1231 0 0 nch w=1u l=180n
M3401 t1233 nw371 vdd vdd pch w=2u l=180n
M3402 t1233 t1231 vdd vdd pch w=2u l=180n
CT1236 t1236 0 0.1f
M3403 t1233 nw371 t1236 0 nch w=1u l=180n
M3404 t1236 t1231 0 0 nch w=1u l=180n
M3405 nw467 t1232 vdd vdd pch w=2u l=180n
M3406 nw467 t1233 vdd vdd pch w=2u l=180n
CT1237 t1237 0 0.1f
M3407 nw467 t1232 t1237 0 nch w=1u l=180n
M3408 t1237 t1233 0 0 nch w=1u l=180n
Cnw467 nw467 0 2f
M3409 nw468 nw406 vdd vdd pch w=2u l=180n
M3410 nw468 nw372 vdd vdd pch w=2u l=180n
CT1238 t1238 0 0.1f
M3411 nw468 nw406 t1238 0 nch w=1u l=180n
M3412 t1238 nw372 0 0 nch w=1u l=180n
Cnw468 nw468 0 2f
M3413 nw469 nw407 0 0 nch w=1u l=180n
M3414 nw469 nw373 0 0 nch w=1u l=180n
CT1239 t1239 0 0.1f
M3415 t1239 nw407 vdd vdd pch w=2u l=180n
M3416 nw469 nw373 t1239 vdd pch w=2u l=180n
Cnw469 nw469 0 2f
CT1240 t1240 0 0.1f
M3417 t1240 nw408 vdd vdd pch w=2u l=180n
M3418 t1240 nw374 vdd vdd pch w=2u l=180n
CT1241 t1241 0 0.1f
M3419 t1240 nw408 t1241 0 nch w=1u l=180n
M3420 t1241 nw374 0 0 nch w=1u l=180n
M3421 nw470 t1240 vdd vdd pch w=2u l=180n
M3422 nw470 t1240 0 0 nch w=1u l=180n
Cnw470 nw470 0 2f
CT1242 t1242 0 0.1f
M3423 t1242 nw409 0 0 nch w=1u l=180n
M3424 t1242 nw375 0 0 nch w=1u l=180n
CT1243 t1243 0 0.1f
M3425 t1243 nw409 vdd vdd pch w=2u l=180n
M3426 t1242 nw375 t1243 vdd pch w=2u l=180n
M3427 nw471 t1242 vdd vdd pch w=2u l=180n
M3428 nw471 t1242 0 0 nch w=1u l=180n
Cnw471 nw471 0 2f
CT1244 t1244 0 0.1f
CT1245 t1245 0 0.1f
CT1246 t1246 0 0.1f
M3429 t1244 nw410 vdd vdd pch w=2u l=180n
M3430 t1244 nw376 vdd vdd pch w=2u l=180n
CT1247 t1247 0 0.1f
M3431 t1244 nw410 t1247 0 nch w=1u l=180n
M3432 t1247 nw376 0 0 nch w=1u l=180n
M3433 t1245 nw410 vdd vdd pch w=2u l=180n
M3434 t1245 t1244 vdd vdd pch w=2u l=180n
CT1248 t1248 0 0.1f
M3435 t1245 nw410 t1248 0 nch w=1u l=180n
M3436 t1248 t1244 0 0 nch w=1u l=180n
M3437 t1246 nw376 vdd vdd pch w=2u l=180n
M3438 t1246 t1244 vdd vdd pch w=2u l=180n
CT1249 t1249 0 0.1f
M3439 t1246 nw376 t1249 0 nch w=1u l=180n
M3440 t1249 t1244 0 0 nch w=1u l=180n
M3441 nw472 t1245 vdd vdd pch w=2u l=180n
M3442 nw472 t1246 vdd vdd pch w=2u l=180n
CT1250 t1250 0 0.1f
M3443 nw472 t1245 t1250 0 nch w=1u l=180n
M3444 t1250 t1246 0 0 nch w=1u l=180n
Cnw472 nw472 0 2f
M3445 nw473 nw411 vdd vdd pch w=2u l=180n
M3446 nw473 nw377 vdd vdd pch w=2u l=180n
CT1251 t1251 0 0.1f
M3447 nw473 nw411 t1251 0 nch w=1u l=180n
M3448 t1251 nw377 0 0 nch w=1u l=180n
Cnw473 nw473 0 2f
M3449 nw474 nw412 0 0 nch w=1u l=180n
M3450 nw474 nw378 0 0 nch w=1u l=180n
CT1252 t1252 0 0.1f
M3451 t1252 nw412 vdd vdd pch w=2u l=180n
M3452 nw474 nw378 t1252 vdd pch w=2u l=180n
Cnw474 nw474 0 2f
CT1253 t1253 0 0.1f
M3453 t1253 nw413 vdd vdd pch w=2u l=180n
M3454 t1253 nw379 vdd vdd pch w=2u l=180n
CT1254 t1254 0 0.1f
M3455 t1253 nw413 t1254 0 nch w=1u l=180n
M3456 t1254 nw379 0 0 nch w=1u l=180n
M3457 nw475 t1253 vdd vdd pch w=2u l=180n
M3458 nw475 t1253 0 0 nch w=1u l=180n
Cnw475 nw475 0 2f
CT1255 t1255 0 0.1f
M3459 t1255 nw414 0 0 nch w=1u l=180n
M3460 t1255 nw380 0 0 nch w=1u l=180n
CT1256 t1256 0 0.1f
M3461 t1256 nw414 vdd vdd pch w=2u l=180n
M3462 t1255 nw380 t1256 vdd pch w=2u l=180n
M3463 nw476 t1255 vdd vdd pch w=2u l=180n
M3464 nw476 t1255 0 0 nch w=1u l=180n
Cnw476 nw476 0 2f
CT1257 t1257 0 0.1f
CT1258 t1258 0 0.1f
CT1259 t1259 0 0.1f
M3465 t1257 nw415 vdd vdd pch w=2u l=180n
M3466 t1257 nw381 vdd vdd pch w=2u l=180n
CT1260 t1260 0 0.1f
M3467 t1257 nw415 t1260 0 nch w=1u l=180n
M3468 t1260 nw381 0 0 nch w=1u l=180n
M3469 t1258 nw415 vdd vdd pch w=2u l=180n
M3470 t1258 t1257 vdd vdd pch w=2u l=180n
CT1261 t1261 0 0.1f
M3471 t1258 nw415 t1261 0 nch w=1u l=180n
M3472 t1261 t1257 0 0 nch w=1u l=180n
M3473 t1259 nw381 vdd vdd pch w=2u l=180n
M3474 t1259 t1257 vdd vdd pch w=2u l=180n
CT1262 t1262 0 0.1f
M3475 t1259 nw381 t1262 0 nch w=1u l=180n
M3476 t1262 t1257 0 0 nch w=1u l=180n
M3477 nw477 t1258 vdd vdd pch w=2u l=180n
M3478 nw477 t1259 vdd vdd pch w=2u l=180n
CT1263 t1263 0 0.1f
M3479 nw477 t1258 t1263 0 nch w=1u l=180n
M3480 t1263 t1259 0 0 nch w=1u l=180n
Cnw477 nw477 0 2f
M3481 nw478 nw416 vdd vdd pch w=2u l=180n
M3482 nw478 nw382 vdd vdd pch w=2u l=180n
CT1264 t1264 0 0.1f
M3483 nw478 nw416 t1264 0 nch w=1u l=180n
M3484 t1264 nw382 0 0 nch w=1u l=180n
Cnw478 nw478 0 2f
M3485 nw479 nw417 0 0 nch w=1u l=180n
M3486 nw479 nw383 0 0 nch w=1u l=180n
CT1265 t1265 0 0.1f
M3487 t1265 nw417 vdd vdd pch w=2u l=180n
M3488 nw479 nw383 t1265 vdd pch w=2u l=180n
Cnw479 nw479 0 2f
CT1266 t1266 0 0.1f
M3489 t1266 nw418 vdd vdd pch w=2u l=180n
M3490 t1266 nw384 vdd vdd pch w=2u l=180n
CT1267 t1267 0 0.1f
M3491 t1266 nw418 t1267 0 nch w=1u l=180n
M3492 t1267 nw384 0 0 nch w=1u l=180n
M3493 nw480 t1266 vdd vdd pch w=2u l=180n
M3494 nw480 t1266 0 0 nch w=1u l=180n
Cnw480 nw480 0 2f
CT1268 t1268 0 0.1f
M3495 t1268 nw419 0 0 nch w=1u l=180n
M3496 t1268 nw385 0 0 nch w=1u l=180n
CT1269 t1269 0 0.1f
M3497 t1269 nw419 vdd vdd pch w=2u l=180n
M3498 t1268 nw385 t1269 vdd pch w=2u l=180n
M3499 nw481 t1268 vdd vdd pch w=2u l=180n
M3500 nw481 t1268 0 0 nch w=1u l=180n
Cnw481 nw481 0 2f
CT1270 t1270 0 0.1f
CT1271 t1271 0 0.1f
CT1272 t1272 0 0.1f
M3501 t1270 nw420 vdd vdd pch w=2u l=180n
M3502 t1270 nw386 vdd vdd pch w=2u l=180n
CT1273 t1273 0 0.1f
M3503 t1270 nw420 t1273 0 nch w=1u l=180n
M3504 t1273 nw386 0 0 nch w=1u l=180n
M3505 t1271 nw420 vdd vdd pch w=2u l=180n
M3506 t1271 t1270 vdd vdd pch w=2u l=180n
CT1274 t1274 0 0.1f
M3507 t1271 nw420 t1274 0 nch w=1u l=180n
M3508 t1274 t1270 0 0 nch w=1u l=180n
M3509 t1272 nw386 vdd vdd pch w=2u l=180n
M3510 t1272 t1270 vdd vdd pch w=2u l=180n
CT1275 t1275 0 0.1f
M3511 t1272 nw386 t1275 0 nch w=1u l=180n
M3512 t1275 t1270 0 0 nch w=1u l=180n
M3513 nw482 t1271 vdd vdd pch w=2u l=180n
M3514 nw482 t1272 vdd vdd pch w=2u l=180n
CT1276 t1276 0 0.1f
M3515 nw482 t1271 t1276 0 nch w=1u l=180n
M3516 t1276 t1272 0 0 nch w=1u l=180n
Cnw482 nw482 0 2f
M3517 nw483 nw421 vdd vdd pch w=2u l=180n
M3518 nw483 nw387 vdd vdd pch w=2u l=180n
CT1277 t1277 0 0.1f
M3519 nw483 nw421 t1277 0 nch w=1u l=180n
M3520 t1277 nw387 0 0 nch w=1u l=180n
Cnw483 nw483 0 2f
M3521 nw484 nw422 0 0 nch w=1u l=180n
M3522 nw484 nw388 0 0 nch w=1u l=180n
CT1278 t1278 0 0.1f
M3523 t1278 nw422 vdd vdd pch w=2u l=180n
M3524 nw484 nw388 t1278 vdd pch w=2u l=180n
Cnw484 nw484 0 2f
CT1279 t1279 0 0.1f
M3525 t1279 nw423 vdd vdd pch w=2u l=180n
M3526 t1279 nw389 vdd vdd pch w=2u l=180n
CT1280 t1280 0 0.1f
M3527 t1279 nw423 t1280 0 nch w=1u l=180n
M3528 t1280 nw389 0 0 nch w=1u l=180n
M3529 nw485 t1279 vdd vdd pch w=2u l=180n
M3530 nw485 t1279 0 0 nch w=1u l=180n
Cnw485 nw485 0 2f
CT1281 t1281 0 0.1f
M3531 t1281 nw424 0 0 nch w=1u l=180n
M3532 t1281 nw390 0 0 nch w=1u l=180n
CT1282 t1282 0 0.1f
M3533 t1282 nw424 vdd vdd pch w=2u l=180n
M3534 t1281 nw390 t1282 vdd pch w=2u l=180n
M3535 nw486 t1281 vdd vdd pch w=2u l=180n
M3536 nw486 t1281 0 0 nch w=1u l=180n
Cnw486 nw486 0 2f
CT1283 t1283 0 0.1f
CT1284 t1284 0 0.1f
CT1285 t1285 0 0.1f
M3537 t1283 nw425 vdd vdd pch w=2u l=180n
M3538 t1283 nw391 vdd vdd pch w=2u l=180n
CT1286 t1286 0 0.1f
M3539 t1283 nw425 t1286 0 nch w=1u l=180n
M3540 t1286 nw391 0 0 nch w=1u l=180n
M3541 t1284 nw425 vdd vdd pch w=2u l=180n
M3542 t1284 t1283 vdd vdd pch w=2u l=180n
CT1287 t1287 0 0.1f
M3543 t1284 nw425 t1287 0 nch w=1u l=180n
M3544 t1287 t1283 0 0 nch w=1u l=180n
M3545 t1285 nw391 vdd vdd pch w=2u l=180n
M3546 t1285 t1283 vdd vdd pch w=2u l=180n
CT1288 t1288 0 0.1f
M3547 t1285 nw391 t1288 0 nch w=1u l=180n
M3548 t1288 t1283 0 0 nch w=1u l=180n
M3549 nw487 t1284 vdd vdd pch w=2u l=180n
M3550 nw487 t1285 vdd vdd pch w=2u l=180n
CT1289 t1289 0 0.1f
M3551 nw487 t1284 t1289 0 nch w=1u l=180n
M3552 t1289 t1285 0 0 nch w=1u l=180n
Cnw487 nw487 0 2f
M3553 nw488 nw426 vdd vdd pch w=2u l=180n
M3554 nw488 nw392 vdd vdd pch w=2u l=180n
CT1290 t1290 0 0.1f
M3555 nw488 nw426 t1290 0 nch w=1u l=180n
M3556 t1290 nw392 0 0 nch w=1u l=180n
Cnw488 nw488 0 2f
M3557 nw489 nw427 0 0 nch w=1u l=180n
M3558 nw489 nw393 0 0 nch w=1u l=180n
CT1291 t1291 0 0.1f
M3559 t1291 nw427 vdd vdd pch w=2u l=180n
M3560 nw489 nw393 t1291 vdd pch w=2u l=180n
Cnw489 nw489 0 2f
CT1292 t1292 0 0.1f
M3561 t1292 nw428 vdd vdd pch w=2u l=180n
M3562 t1292 nw394 vdd vdd pch w=2u l=180n
CT1293 t1293 0 0.1f
M3563 t1292 nw428 t1293 0 nch w=1u l=180n
M3564 t1293 nw394 0 0 nch w=1u l=180n
M3565 nw490 t1292 vdd vdd pch w=2u l=180n
M3566 nw490 t1292 0 0 nch w=1u l=180n
Cnw490 nw490 0 2f
CT1294 t1294 0 0.1f
M3567 t1294 nw429 0 0 nch w=1u l=180n
M3568 t1294 nw395 0 0 nch w=1u l=180n
CT1295 t1295 0 0.1f
M3569 t1295 nw429 vdd vdd pch w=2u l=180n
M3570 t1294 nw395 t1295 vdd pch w=2u l=180n
M3571 nw491 t1294 vdd vdd pch w=2u l=180n
M3572 nw491 t1294 0 0 nch w=1u l=180n
Cnw491 nw491 0 2f
CT1296 t1296 0 0.1f
CT1297 t1297 0 0.1f
CT1298 t1298 0 0.1f
M3573 t1296 nw430 vdd vdd pch w=2u l=180n
M3574 t1296 nw396 vdd vdd pch w=2u l=180n
CT1299 t1299 0 0.1f
M3575 t1296 nw430 t1299 0 nch w=1u l=180n
M3576 t1299 nw396 0 0 nch w=1u l=180n
M3577 t1297 nw430 vdd vdd pch w=2u l=180n
M3578 t1297 t1296 vdd vdd pch w=2u l=180n
CT1300 t1300 0 0.1f
M3579 t1297 nw430 t1300 0 nch w=1u l=180n
M3580 t1300 t1296 0 0 nch w=1u l=180n
M3581 t1298 nw396 vdd vdd pch w=2u l=180n
M3582 t1298 t1296 vdd vdd pch w=2u l=180n
CT1301 t1301 0 0.1f
M3583 t1298 nw396 t1301 0 nch w=1u l=180n
M3584 t1301 t1296 0 0 nch w=1u l=180n
M3585 nw492 t1297 vdd vdd pch w=2u l=180n
M3586 nw492 t1298 vdd vdd pch w=2u l=180n
CT1302 t1302 0 0.1f
M3587 nw492 t1297 t1302 0 nch w=1u l=180n
M3588 t1302 t1298 0 0 nch w=1u l=180n
Cnw492 nw492 0 2f
M3589 nw493 nw431 vdd vdd pch w=2u l=180n
M3590 nw493 nw397 vdd vdd pch w=2u l=180n
CT1303 t1303 0 0.1f
M3591 nw493 nw431 t1303 0 nch w=1u l=180n
M3592 t1303 nw397 0 0 nch w=1u l=180n
Cnw493 nw493 0 2f
M3593 nw494 nw432 0 0 nch w=1u l=180n
M3594 nw494 nw398 0 0 nch w=1u l=180n
CT1304 t1304 0 0.1f
M3595 t1304 nw432 vdd vdd pch w=2u l=180n
M3596 nw494 nw398 t1304 vdd pch w=2u l=180n
Cnw494 nw494 0 2f
CT1305 t1305 0 0.1f
M3597 t1305 nw433 vdd vdd pch w=2u l=180n
M3598 t1305 nw399 vdd vdd pch w=2u l=180n
CT1306 t1306 0 0.1f
M3599 t1305 nw433 t1306 0 nch w=1u l=180n
M3600 t1306 nw399 0 0 nch w=1u l=180n
M3601 nw495 t1305 vdd vdd pch w=2u l=180n
M3602 nw495 t1305 0 0 nch w=1u l=180n
Cnw495 nw495 0 2f
CT1307 t1307 0 0.1f
M3603 t1307 nw434 0 0 nch w=1u l=180n
M3604 t1307 nw400 0 0 nch w=1u l=180n
CT1308 t1308 0 0.1f
M3605 t1308 nw434 vdd vdd pch w=2u l=180n
M3606 t1307 nw400 t1308 vdd pch w=2u l=180n
M3607 nw496 t1307 vdd vdd pch w=2u l=180n
M3608 nw496 t1307 0 0 nch w=1u l=180n
Cnw496 nw496 0 2f
CT1309 t1309 0 0.1f
CT1310 t1310 0 0.1f
CT1311 t1311 0 0.1f
M3609 t1309 nw435 vdd vdd pch w=2u l=180n
M3610 t1309 nw401 vdd vdd pch w=2u l=180n
CT1312 t1312 0 0.1f
M3611 t1309 nw435 t1312 0 nch w=1u l=180n
M3612 t1312 nw401 0 0 nch w=1u l=180n
M3613 t1310 nw435 vdd vdd pch w=2u l=180n
M3614 t1310 t1309 vdd vdd pch w=2u l=180n
CT1313 t1313 0 0.1f
M3615 t1310 nw435 t1313 0 nch w=1u l=180n
M3616 t1313 t1309 0 0 nch w=1u l=180n
M3617 t1311 nw401 vdd vdd pch w=2u l=180n
M3618 t1311 t1309 vdd vdd pch w=2u l=180n
CT1314 t1314 0 0.1f
M3619 t1311 nw401 t1314 0 nch w=1u l=180n
M3620 t1314 t1309 0 0 nch w=1u l=180n
M3621 nw497 t1310 vdd vdd pch w=2u l=180n
M3622 nw497 t1311 vdd vdd pch w=2u l=180n
CT1315 t1315 0 0.1f
M3623 nw497 t1310 t1315 0 nch w=1u l=180n
M3624 t1315 t1311 0 0 nch w=1u l=180n
Cnw497 nw497 0 2f
M3625 nw498 nw436 vdd vdd pch w=2u l=180n
M3626 nw498 nw402 vdd vdd pch w=2u l=180n
CT1316 t1316 0 0.1f
M3627 nw498 nw436 t1316 0 nch w=1u l=180n
M3628 t1316 nw402 0 0 nch w=1u l=180n
Cnw498 nw498 0 2f
M3629 nw499 nw437 0 0 nch w=1u l=180n
M3630 nw499 nw403 0 0 nch w=1u l=180n
CT1317 t1317 0 0.1f
M3631 t1317 nw437 vdd vdd pch w=2u l=180n
M3632 nw499 nw403 t1317 vdd pch w=2u l=180n
Cnw499 nw499 0 2f
CT1318 t1318 0 0.1f
M3633 t1318 nw438 vdd vdd pch w=2u l=180n
M3634 t1318 nw404 vdd vdd pch w=2u l=180n
CT1319 t1319 0 0.1f
M3635 t1318 nw438 t1319 0 nch w=1u l=180n
M3636 t1319 nw404 0 0 nch w=1u l=180n
M3637 nw500 t1318 vdd vdd pch w=2u l=180n
M3638 nw500 t1318 0 0 nch w=1u l=180n
Cnw500 nw500 0 2f
CT1320 t1320 0 0.1f
M3639 t1320 nw439 0 0 nch w=1u l=180n
M3640 t1320 nw405 0 0 nch w=1u l=180n
CT1321 t1321 0 0.1f
M3641 t1321 nw439 vdd vdd pch w=2u l=180n
M3642 t1320 nw405 t1321 vdd pch w=2u l=180n
M3643 nw501 t1320 vdd vdd pch w=2u l=180n
M3644 nw501 t1320 0 0 nch w=1u l=180n
Cnw501 nw501 0 2f
CT1322 t1322 0 0.1f
CT1323 t1323 0 0.1f
CT1324 t1324 0 0.1f
M3645 t1322 nw440 vdd vdd pch w=2u l=180n
M3646 t1322 nw406 vdd vdd pch w=2u l=180n
CT1325 t1325 0 0.1f
M3647 t1322 nw440 t1325 0 nch w=1u l=180n
M3648 t1325 nw406 0 0 nch w=1u l=180n
M3649 t1323 nw440 vdd vdd pch w=2u l=180n
M3650 t1323 t1322 vdd vdd pch w=2u l=180n
CT1326 t1326 0 0.1f
M3651 t1323 nw440 t1326 0 nch w=1u l=180n
M3652 t1326 t1322 0 0 nch w=1u l=180n
M3653 t1324 nw406 vdd vdd pch w=2u l=180n
M3654 t1324 t1322 vdd vdd pch w=2u l=180n
CT1327 t1327 0 0.1f
M3655 t1324 nw406 t1327 0 nch w=1u l=180n
M3656 t1327 t1322 0 0 nch w=1u l=180n
M3657 nw502 t1323 vdd vdd pch w=2u l=180n
M3658 nw502 t1324 vdd vdd pch w=2u l=180n
CT1328 t1328 0 0.1f
M3659 nw502 t1323 t1328 0 nch w=1u l=180n
M3660 t1328 t1324 0 0 nch w=1u l=180n
Cnw502 nw502 0 2f
M3661 nw503 nw441 vdd vdd pch w=2u l=180n
M3662 nw503 nw407 vdd vdd pch w=2u l=180n
CT1329 t1329 0 0.1f
M3663 nw503 nw441 t1329 0 nch w=1u l=180n
M3664 t1329 nw407 0 0 nch w=1u l=180n
Cnw503 nw503 0 2f
M3665 nw504 nw442 0 0 nch w=1u l=180n
M3666 nw504 nw408 0 0 nch w=1u l=180n
CT1330 t1330 0 0.1f
M3667 t1330 nw442 vdd vdd pch w=2u l=180n
M3668 nw504 nw408 t1330 vdd pch w=2u l=180n
Cnw504 nw504 0 2f
CT1331 t1331 0 0.1f
M3669 t1331 nw443 vdd vdd pch w=2u l=180n
M3670 t1331 nw409 vdd vdd pch w=2u l=180n
CT1332 t1332 0 0.1f
M3671 t1331 nw443 t1332 0 nch w=1u l=180n
M3672 t1332 nw409 0 0 nch w=1u l=180n
M3673 nw505 t1331 vdd vdd pch w=2u l=180n
M3674 nw505 t1331 0 0 nch w=1u l=180n
Cnw505 nw505 0 2f
CT1333 t1333 0 0.1f
M3675 t1333 nw444 0 0 nch w=1u l=180n
M3676 t1333 nw410 0 0 nch w=1u l=180n
CT1334 t1334 0 0.1f
M3677 t1334 nw444 vdd vdd pch w=2u l=180n
M3678 t1333 nw410 t1334 vdd pch w=2u l=180n
M3679 nw506 t1333 vdd vdd pch w=2u l=180n
M3680 nw506 t1333 0 0 nch w=1u l=180n
Cnw506 nw506 0 2f
CT1335 t1335 0 0.1f
CT1336 t1336 0 0.1f
CT1337 t1337 0 0.1f
M3681 t1335 nw445 vdd vdd pch w=2u l=180n
M3682 t1335 nw411 vdd vdd pch w=2u l=180n
CT1338 t1338 0 0.1f
M3683 t1335 nw445 t1338 0 nch w=1u l=180n
M3684 t1338 nw411 0 0 nch w=1u l=180n
M3685 t1336 nw445 vdd vdd pch w=2u l=180n
M3686 t1336 t1335 vdd vdd pch w=2u l=180n
CT1339 t1339 0 0.1f
M3687 t1336 nw445 t1339 0 nch w=1u l=180n
M3688 t1339 t1335 0 0 nch w=1u l=180n
M3689 t1337 nw411 vdd vdd pch w=2u l=180n
M3690 t1337 t1335 vdd vdd pch w=2u l=180n
CT1340 t1340 0 0.1f
M3691 t1337 nw411 t1340 0 nch w=1u l=180n
M3692 t1340 t1335 0 0 nch w=1u l=180n
M3693 nw507 t1336 vdd vdd pch w=2u l=180n
M3694 nw507 t1337 vdd vdd pch w=2u l=180n
CT1341 t1341 0 0.1f
M3695 nw507 t1336 t1341 0 nch w=1u l=180n
M3696 t1341 t1337 0 0 nch w=1u l=180n
Cnw507 nw507 0 2f
M3697 nw508 nw446 vdd vdd pch w=2u l=180n
M3698 nw508 nw412 vdd vdd pch w=2u l=180n
CT1342 t1342 0 0.1f
M3699 nw508 nw446 t1342 0 nch w=1u l=180n
M3700 t1342 nw412 0 0 nch w=1u l=180n
Cnw508 nw508 0 2f
M3701 nw509 nw447 0 0 nch w=1u l=180n
M3702 nw509 nw413 0 0 nch w=1u l=180n
CT1343 t1343 0 0.1f
M3703 t1343 nw447 vdd vdd pch w=2u l=180n
M3704 nw509 nw413 t1343 vdd pch w=2u l=180n
Cnw509 nw509 0 2f
CT1344 t1344 0 0.1f
M3705 t1344 nw448 vdd vdd pch w=2u l=180n
M3706 t1344 nw414 vdd vdd pch w=2u l=180n
CT1345 t1345 0 0.1f
M3707 t1344 nw448 t1345 0 nch w=1u l=180n
M3708 t1345 nw414 0 0 nch w=1u l=180n
M3709 nw510 t1344 vdd vdd pch w=2u l=180n
M3710 nw510 t1344 0 0 nch w=1u l=180n
Cnw510 nw510 0 2f
CT1346 t1346 0 0.1f
M3711 t1346 nw449 0 0 nch w=1u l=180n
M3712 t1346 nw415 0 0 nch w=1u l=180n
CT1347 t1347 0 0.1f
M3713 t1347 nw449 vdd vdd pch w=2u l=180n
M3714 t1346 nw415 t1347 vdd pch w=2u l=180n
M3715 nw511 t1346 vdd vdd pch w=2u l=180n
M3716 nw511 t1346 0 0 nch w=1u l=180n
Cnw511 nw511 0 2f
CT1348 t1348 0 0.1f
CT1349 t1349 0 0.1f
CT1350 t1350 0 0.1f
M3717 t1348 nw450 vdd vdd pch w=2u l=180n
M3718 t1348 nw416 vdd vdd pch w=2u l=180n
CT1351 t1351 0 0.1f
M3719 t1348 nw450 t1351 0 nch w=1u l=180n
M3720 t1351 nw416 0 0 nch w=1u l=180n
M3721 t1349 nw450 vdd vdd pch w=2u l=180n
M3722 t1349 t1348 vdd vdd pch w=2u l=180n
CT1352 t1352 0 0.1f
M3723 t1349 nw450 t1352 0 nch w=1u l=180n
M3724 t1352 t1348 0 0 nch w=1u l=180n
M3725 t1350 nw416 vdd vdd pch w=2u l=180n
M3726 t1350 t1348 vdd vdd pch w=2u l=180n
CT1353 t1353 0 0.1f
M3727 t1350 nw416 t1353 0 nch w=1u l=180n
M3728 t1353 t1348 0 0 nch w=1u l=180n
M3729 nw512 t1349 vdd vdd pch w=2u l=180n
M3730 nw512 t1350 vdd vdd pch w=2u l=180n
CT1354 t1354 0 0.1f
M3731 nw512 t1349 t1354 0 nch w=1u l=180n
M3732 t1354 t1350 0 0 nch w=1u l=180n
Cnw512 nw512 0 2f
M3733 nw513 nw451 vdd vdd pch w=2u l=180n
M3734 nw513 nw417 vdd vdd pch w=2u l=180n
CT1355 t1355 0 0.1f
M3735 nw513 nw451 t1355 0 nch w=1u l=180n
M3736 t1355 nw417 0 0 nch w=1u l=180n
Cnw513 nw513 0 2f
M3737 nw514 nw452 0 0 nch w=1u l=180n
M3738 nw514 nw418 0 0 nch w=1u l=180n
CT1356 t1356 0 0.1f
M3739 t1356 nw452 vdd vdd pch w=2u l=180n
M3740 nw514 nw418 t1356 vdd pch w=2u l=180n
Cnw514 nw514 0 2f
CT1357 t1357 0 0.1f
M3741 t1357 nw453 vdd vdd pch w=2u l=180n
M3742 t1357 nw419 vdd vdd pch w=2u l=180n
CT1358 t1358 0 0.1f
M3743 t1357 nw453 t1358 0 nch w=1u l=180n
M3744 t1358 nw419 0 0 nch w=1u l=180n
M3745 nw515 t1357 vdd vdd pch w=2u l=180n
M3746 nw515 t1357 0 0 nch w=1u l=180n
Cnw515 nw515 0 2f
CT1359 t1359 0 0.1f
M3747 t1359 nw454 0 0 nch w=1u l=180n
M3748 t1359 nw420 0 0 nch w=1u l=180n
CT1360 t1360 0 0.1f
M3749 t1360 nw454 vdd vdd pch w=2u l=180n
M3750 t1359 nw420 t1360 vdd pch w=2u l=180n
M3751 nw516 t1359 vdd vdd pch w=2u l=180n
M3752 nw516 t1359 0 0 nch w=1u l=180n
Cnw516 nw516 0 2f
CT1361 t1361 0 0.1f
CT1362 t1362 0 0.1f
CT1363 t1363 0 0.1f
M3753 t1361 nw455 vdd vdd pch w=2u l=180n
M3754 t1361 nw421 vdd vdd pch w=2u l=180n
CT1364 t1364 0 0.1f
M3755 t1361 nw455 t1364 0 nch w=1u l=180n
M3756 t1364 nw421 0 0 nch w=1u l=180n
M3757 t1362 nw455 vdd vdd pch w=2u l=180n
M3758 t1362 t1361 vdd vdd pch w=2u l=180n
CT1365 t1365 0 0.1f
M3759 t1362 nw455 t1365 0 nch w=1u l=180n
M3760 t1365 t1361 0 0 nch w=1u l=180n
M3761 t1363 nw421 vdd vdd pch w=2u l=180n
M3762 t1363 t1361 vdd vdd pch w=2u l=180n
CT1366 t1366 0 0.1f
M3763 t1363 nw421 t1366 0 nch w=1u l=180n
M3764 t1366 t1361 0 0 nch w=1u l=180n
M3765 nw517 t1362 vdd vdd pch w=2u l=180n
M3766 nw517 t1363 vdd vdd pch w=2u l=180n
CT1367 t1367 0 0.1f
M3767 nw517 t1362 t1367 0 nch w=1u l=180n
M3768 t1367 t1363 0 0 nch w=1u l=180n
Cnw517 nw517 0 2f
M3769 nw518 nw456 vdd vdd pch w=2u l=180n
M3770 nw518 nw422 vdd vdd pch w=2u l=180n
CT1368 t1368 0 0.1f
M3771 nw518 nw456 t1368 0 nch w=1u l=180n
M3772 t1368 nw422 0 0 nch w=1u l=180n
Cnw518 nw518 0 2f
M3773 nw519 nw457 0 0 nch w=1u l=180n
M3774 nw519 nw423 0 0 nch w=1u l=180n
CT1369 t1369 0 0.1f
M3775 t1369 nw457 vdd vdd pch w=2u l=180n
M3776 nw519 nw423 t1369 vdd pch w=2u l=180n
Cnw519 nw519 0 2f
CT1370 t1370 0 0.1f
M3777 t1370 nw458 vdd vdd pch w=2u l=180n
M3778 t1370 nw424 vdd vdd pch w=2u l=180n
CT1371 t1371 0 0.1f
M3779 t1370 nw458 t1371 0 nch w=1u l=180n
M3780 t1371 nw424 0 0 nch w=1u l=180n
M3781 nw520 t1370 vdd vdd pch w=2u l=180n
M3782 nw520 t1370 0 0 nch w=1u l=180n
Cnw520 nw520 0 2f
CT1372 t1372 0 0.1f
M3783 t1372 nw459 0 0 nch w=1u l=180n
M3784 t1372 nw425 0 0 nch w=1u l=180n
CT1373 t1373 0 0.1f
M3785 t1373 nw459 vdd vdd pch w=2u l=180n
M3786 t1372 nw425 t1373 vdd pch w=2u l=180n
M3787 nw521 t1372 vdd vdd pch w=2u l=180n
M3788 nw521 t1372 0 0 nch w=1u l=180n
Cnw521 nw521 0 2f
CT1374 t1374 0 0.1f
CT1375 t1375 0 0.1f
CT1376 t1376 0 0.1f
M3789 t1374 nw460 vdd vdd pch w=2u l=180n
M3790 t1374 nw426 vdd vdd pch w=2u l=180n
CT1377 t1377 0 0.1f
M3791 t1374 nw460 t1377 0 nch w=1u l=180n
M3792 t1377 nw426 0 0 nch w=1u l=180n
M3793 t1375 nw460 vdd vdd pch w=2u l=180n
M3794 t1375 t1374 vdd vdd pch w=2u l=180n
CT1378 t1378 0 0.1f
M3795 t1375 nw460 t1378 0 nch w=1u l=180n
M3796 t1378 t1374 0 0 nch w=1u l=180n
M3797 t1376 nw426 vdd vdd pch w=2u l=180n
M3798 t1376 t1374 vdd vdd pch w=2u l=180n
CT1379 t1379 0 0.1f
M3799 t1376 nw426 t1379 0 nch w=1u l=180n
M3800 t1379 t1374 0 0 nch w=1u l=180n
M3801 nw522 t1375 vdd vdd pch w=2u l=180n
M3802 nw522 t1376 vdd vdd pch w=2u l=180n
CT1380 t1380 0 0.1f
M3803 nw522 t1375 t1380 0 nch w=1u l=180n
M3804 t1380 t1376 0 0 nch w=1u l=180n
Cnw522 nw522 0 2f
M3805 nw523 nw461 vdd vdd pch w=2u l=180n
M3806 nw523 nw427 vdd vdd pch w=2u l=180n
CT1381 t1381 0 0.1f
M3807 nw523 nw461 t1381 0 nch w=1u l=180n
M3808 t1381 nw427 0 0 nch w=1u l=180n
Cnw523 nw523 0 2f
M3809 nw524 nw462 0 0 nch w=1u l=180n
M3810 nw524 nw428 0 0 nch w=1u l=180n
CT1382 t1382 0 0.1f
M3811 t1382 nw462 vdd vdd pch w=2u l=180n
M3812 nw524 nw428 t1382 vdd pch w=2u l=180n
Cnw524 nw524 0 2f
CT1383 t1383 0 0.1f
M3813 t1383 nw463 vdd vdd pch w=2u l=180n
M3814 t1383 nw429 vdd vdd pch w=2u l=180n
CT1384 t1384 0 0.1f
M3815 t1383 nw463 t1384 0 nch w=1u l=180n
M3816 t1384 nw429 0 0 nch w=1u l=180n
M3817 nw525 t1383 vdd vdd pch w=2u l=180n
M3818 nw525 t1383 0 0 nch w=1u l=180n
Cnw525 nw525 0 2f
CT1385 t1385 0 0.1f
M3819 t1385 nw464 0 0 nch w=1u l=180n
M3820 t1385 nw430 0 0 nch w=1u l=180n
CT1386 t1386 0 0.1f
M3821 t1386 nw464 vdd vdd pch w=2u l=180n
M3822 t1385 nw430 t1386 vdd pch w=2u l=180n
M3823 nw526 t1385 vdd vdd pch w=2u l=180n
M3824 nw526 t1385 0 0 nch w=1u l=180n
Cnw526 nw526 0 2f
CT1387 t1387 0 0.1f
CT1388 t1388 0 0.1f
CT1389 t1389 0 0.1f
M3825 t1387 nw465 vdd vdd pch w=2u l=180n
M3826 t1387 nw431 vdd vdd pch w=2u l=180n
CT1390 t1390 0 0.1f
M3827 t1387 nw465 t1390 0 nch w=1u l=180n
M3828 t1390 nw431 0 0 nch w=1u l=180n
M3829 t1388 nw465 vdd vdd pch w=2u l=180n
M3830 t1388 t1387 vdd vdd pch w=2u l=180n
CT1391 t1391 0 0.1f
M3831 t1388 nw465 t1391 0 nch w=1u l=180n
M3832 t1391 t1387 0 0 nch w=1u l=180n
M3833 t1389 nw431 vdd vdd pch w=2u l=180n
M3834 t1389 t1387 vdd vdd pch w=2u l=180n
CT1392 t1392 0 0.1f
M3835 t1389 nw431 t1392 0 nch w=1u l=180n
M3836 t1392 t1387 0 0 nch w=1u l=180n
M3837 nw527 t1388 vdd vdd pch w=2u l=180n
M3838 nw527 t1389 vdd vdd pch w=2u l=180n
CT1393 t1393 0 0.1f
M3839 nw527 t1388 t1393 0 nch w=1u l=180n
M3840 t1393 t1389 0 0 nch w=1u l=180n
Cnw527 nw527 0 2f
M3841 nw528 nw466 vdd vdd pch w=2u l=180n
M3842 nw528 nw432 vdd vdd pch w=2u l=180n
CT1394 t1394 0 0.1f
M3843 nw528 nw466 t1394 0 nch w=1u l=180n
M3844 t1394 nw432 0 0 nch w=1u l=180n
Cnw528 nw528 0 2f
M3845 nw529 nw467 0 0 nch w=1u l=180n
M3846 nw529 nw433 0 0 nch w=1u l=180n
CT1395 t1395 0 0.1f
M3847 t1395 nw467 vdd vdd pch w=2u l=180n
M3848 nw529 nw433 t1395 vdd pch w=2u l=180n
Cnw529 nw529 0 2f
CT1396 t1396 0 0.1f
M3849 t1396 nw468 vdd vdd pch w=2u l=180n
M3850 t1396 nw434 vdd vdd pch w=2u l=180n
CT1397 t1397 0 0.1f
M3851 t1396 nw468 t1397 0 nch w=1u l=180n
M3852 t1397 nw434 0 0 nch w=1u l=180n
M3853 nw530 t1396 vdd vdd pch w=2u l=180n
M3854 nw530 t1396 0 0 nch w=1u l=180n
Cnw530 nw530 0 2f
CT1398 t1398 0 0.1f
M3855 t1398 nw469 0 0 nch w=1u l=180n
M3856 t1398 nw435 0 0 nch w=1u l=180n
CT1399 t1399 0 0.1f
M3857 t1399 nw469 vdd vdd pch w=2u l=180n
M3858 t1398 nw435 t1399 vdd pch w=2u l=180n
M3859 nw531 t1398 vdd vdd pch w=2u l=180n
M3860 nw531 t1398 0 0 nch w=1u l=180n
Cnw531 nw531 0 2f
CT1400 t1400 0 0.1f
CT1401 t1401 0 0.1f
CT1402 t1402 0 0.1f
M3861 t1400 nw470 vdd vdd pch w=2u l=180n
M3862 t1400 nw436 vdd vdd pch w=2u l=180n
CT1403 t1403 0 0.1f
M3863 t1400 nw470 t1403 0 nch w=1u l=180n
M3864 t1403 nw436 0 0 nch w=1u l=180n
M3865 t1401 nw470 vdd vdd pch w=2u l=180n
M3866 t1401 t1400 vdd vdd pch w=2u l=180n
CT1404 t1404 0 0.1f
M3867 t1401 nw470 t1404 0 nch w=1u l=180n
M3868 t1404 t1400 0 0 nch w=1u l=180n
M3869 t1402 nw436 vdd vdd pch w=2u l=180n
M3870 t1402 t1400 vdd vdd pch w=2u l=180n
CT1405 t1405 0 0.1f
M3871 t1402 nw436 t1405 0 nch w=1u l=180n
M3872 t1405 t1400 0 0 nch w=1u l=180n
M3873 nw532 t1401 vdd vdd pch w=2u l=180n
M3874 nw532 t1402 vdd vdd pch w=2u l=180n
CT1406 t1406 0 0.1f
M3875 nw532 t1401 t1406 0 nch w=1u l=180n
M3876 t1406 t1402 0 0 nch w=1u l=180n
Cnw532 nw532 0 2f
M3877 nw533 nw471 vdd vdd pch w=2u l=180n
M3878 nw533 nw437 vdd vdd pch w=2u l=180n
CT1407 t1407 0 0.1f
M3879 nw533 nw471 t1407 0 nch w=1u l=180n
M3880 t1407 nw437 0 0 nch w=1u l=180n
Cnw533 nw533 0 2f
M3881 nw534 nw472 0 0 nch w=1u l=180n
M3882 nw534 nw438 0 0 nch w=1u l=180n
CT1408 t1408 0 0.1f
M3883 t1408 nw472 vdd vdd pch w=2u l=180n
M3884 nw534 nw438 t1408 vdd pch w=2u l=180n
Cnw534 nw534 0 2f
CT1409 t1409 0 0.1f
M3885 t1409 nw473 vdd vdd pch w=2u l=180n
M3886 t1409 nw439 vdd vdd pch w=2u l=180n
CT1410 t1410 0 0.1f
M3887 t1409 nw473 t1410 0 nch w=1u l=180n
M3888 t1410 nw439 0 0 nch w=1u l=180n
M3889 nw535 t1409 vdd vdd pch w=2u l=180n
M3890 nw535 t1409 0 0 nch w=1u l=180n
Cnw535 nw535 0 2f
CT1411 t1411 0 0.1f
M3891 t1411 nw474 0 0 nch w=1u l=180n
M3892 t1411 nw440 0 0 nch w=1u l=180n
CT1412 t1412 0 0.1f
M3893 t1412 nw474 vdd vdd pch w=2u l=180n
M3894 t1411 nw440 t1412 vdd pch w=2u l=180n
M3895 nw536 t1411 vdd vdd pch w=2u l=180n
M3896 nw536 t1411 0 0 nch w=1u l=180n
Cnw536 nw536 0 2f
CT1413 t1413 0 0.1f
CT1414 t1414 0 0.1f
CT1415 t1415 0 0.1f
M3897 t1413 nw475 vdd vdd pch w=2u l=180n
M3898 t1413 nw441 vdd vdd pch w=2u l=180n
CT1416 t1416 0 0.1f
M3899 t1413 nw475 t1416 0 nch w=1u l=180n
M3900 t1416 nw441 0 0 nch w=1u l=180n
M3901 t1414 nw475 vdd vdd pch w=2u l=180n
M3902 t1414 t1413 vdd vdd pch w=2u l=180n
CT1417 t1417 0 0.1f
M3903 t1414 nw475 t1417 0 nch w=1u l=180n
M3904 t1417 t1413 0 0 nch w=1u l=180n
M3905 t1415 nw441 vdd vdd pch w=2u l=180n
M3906 t1415 t1413 vdd vdd pch w=2u l=180n
CT1418 t1418 0 0.1f
M3907 t1415 nw441 t1418 0 nch w=1u l=180n
M3908 t1418 t1413 0 0 nch w=1u l=180n
M3909 nw537 t1414 vdd vdd pch w=2u l=180n
M3910 nw537 t1415 vdd vdd pch w=2u l=180n
CT1419 t1419 0 0.1f
M3911 nw537 t1414 t1419 0 nch w=1u l=180n
M3912 t1419 t1415 0 0 nch w=1u l=180n
Cnw537 nw537 0 2f
M3913 nw538 nw476 vdd vdd pch w=2u l=180n
M3914 nw538 nw442 vdd vdd pch w=2u l=180n
CT1420 t1420 0 0.1f
M3915 nw538 nw476 t1420 0 nch w=1u l=180n
M3916 t1420 nw442 0 0 nch w=1u l=180n
Cnw538 nw538 0 2f
M3917 nw539 nw477 0 0 nch w=1u l=180n
M3918 nw539 nw443 0 0 nch w=1u l=180n
CT1421 t1421 0 0.1f
M3919 t1421 nw477 vdd vdd pch w=2u l=180n
M3920 nw539 nw443 t1421 vdd pch w=2u l=180n
Cnw539 nw539 0 2f
CT1422 t1422 0 0.1f
M3921 t1422 nw478 vdd vdd pch w=2u l=180n
M3922 t1422 nw444 vdd vdd pch w=2u l=180n
CT1423 t1423 0 0.1f
M3923 t1422 nw478 t1423 0 nch w=1u l=180n
M3924 t1423 nw444 0 0 nch w=1u l=180n
M3925 nw540 t1422 vdd vdd pch w=2u l=180n
M3926 nw540 t1422 0 0 nch w=1u l=180n
Cnw540 nw540 0 2f
CT1424 t1424 0 0.1f
M3927 t1424 nw479 0 0 nch w=1u l=180n
M3928 t1424 nw445 0 0 nch w=1u l=180n
CT1425 t1425 0 0.1f
M3929 t1425 nw479 vdd vdd pch w=2u l=180n
M3930 t1424 nw445 t1425 vdd pch w=2u l=180n
M3931 nw541 t1424 vdd vdd pch w=2u l=180n
M3932 nw541 t1424 0 0 nch w=1u l=180n
Cnw541 nw541 0 2f
CT1426 t1426 0 0.1f
CT1427 t1427 0 0.1f
CT1428 t1428 0 0.1f
M3933 t1426 nw480 vdd vdd pch w=2u l=180n
M3934 t1426 nw446 vdd vdd pch w=2u l=180n
CT1429 t1429 0 0.1f
M3935 t1426 nw480 t1429 0 nch w=1u l=180n
M3936 t1429 nw446 0 0 nch w=1u l=180n
M3937 t1427 nw480 vdd vdd pch w=2u l=180n
M3938 t1427 t1426 vdd vdd pch w=2u l=180n
CT1430 t1430 0 0.1f
M3939 t1427 nw480 t1430 0 nch w=1u l=180n
M3940 t1430 t1426 0 0 nch w=1u l=180n
M3941 t1428 nw446 vdd vdd pch w=2u l=180n
M3942 t1428 t1426 vdd vdd pch w=2u l=180n
CT1431 t1431 0 0.1f
M3943 t1428 nw446 t1431 0 nch w=1u l=180n
M3944 t1431 t1426 0 0 nch w=1u l=180n
M3945 nw542 t1427 vdd vdd pch w=2u l=180n
M3946 nw542 t1428 vdd vdd pch w=2u l=180n
CT1432 t1432 0 0.1f
M3947 nw542 t1427 t1432 0 nch w=1u l=180n
M3948 t1432 t1428 0 0 nch w=1u l=180n
Cnw542 nw542 0 2f
M3949 nw543 nw481 vdd vdd pch w=2u l=180n
M3950 nw543 nw447 vdd vdd pch w=2u l=180n
CT1433 t1433 0 0.1f
M3951 nw543 nw481 t1433 0 nch w=1u l=180n
M3952 t1433 nw447 0 0 nch w=1u l=180n
Cnw543 nw543 0 2f
M3953 nw544 nw482 0 0 nch w=1u l=180n
M3954 nw544 nw448 0 0 nch w=1u l=180n
CT1434 t1434 0 0.1f
M3955 t1434 nw482 vdd vdd pch w=2u l=180n
M3956 nw544 nw448 t1434 vdd pch w=2u l=180n
Cnw544 nw544 0 2f
CT1435 t1435 0 0.1f
M3957 t1435 nw483 vdd vdd pch w=2u l=180n
M3958 t1435 nw449 vdd vdd pch w=2u l=180n
CT1436 t1436 0 0.1f
M3959 t1435 nw483 t1436 0 nch w=1u l=180n
M3960 t1436 nw449 0 0 nch w=1u l=180n
M3961 nw545 t1435 vdd vdd pch w=2u l=180n
M3962 nw545 t1435 0 0 nch w=1u l=180n
Cnw545 nw545 0 2f
CT1437 t1437 0 0.1f
M3963 t1437 nw484 0 0 nch w=1u l=180n
M3964 t1437 nw450 0 0 nch w=1u l=180n
CT1438 t1438 0 0.1f
M3965 t1438 nw484 vdd vdd pch w=2u l=180n
M3966 t1437 nw450 t1438 vdd pch w=2u l=180n
M3967 nw546 t1437 vdd vdd pch w=2u l=180n
M3968 nw546 t1437 0 0 nch w=1u l=180n
Cnw546 nw546 0 2f
CT1439 t1439 0 0.1f
CT1440 t1440 0 0.1f
CT1441 t1441 0 0.1f
M3969 t1439 nw485 vdd vdd pch w=2u l=180n
M3970 t1439 nw451 vdd vdd pch w=2u l=180n
CT1442 t1442 0 0.1f
M3971 t1439 nw485 t1442 0 nch w=1u l=180n
M3972 t1442 nw451 0 0 nch w=1u l=180n
M3973 t1440 nw485 vdd vdd pch w=2u l=180n
M3974 t1440 t1439 vdd vdd pch w=2u l=180n
CT1443 t1443 0 0.1f
M3975 t1440 nw485 t1443 0 nch w=1u l=180n
M3976 t1443 t1439 0 0 nch w=1u l=180n
M3977 t1441 nw451 vdd vdd pch w=2u l=180n
M3978 t1441 t1439 vdd vdd pch w=2u l=180n
CT1444 t1444 0 0.1f
M3979 t1441 nw451 t1444 0 nch w=1u l=180n
M3980 t1444 t1439 0 0 nch w=1u l=180n
M3981 nw547 t1440 vdd vdd pch w=2u l=180n
M3982 nw547 t1441 vdd vdd pch w=2u l=180n
CT1445 t1445 0 0.1f
M3983 nw547 t1440 t1445 0 nch w=1u l=180n
M3984 t1445 t1441 0 0 nch w=1u l=180n
Cnw547 nw547 0 2f
M3985 nw548 nw486 vdd vdd pch w=2u l=180n
M3986 nw548 nw452 vdd vdd pch w=2u l=180n
CT1446 t1446 0 0.1f
M3987 nw548 nw486 t1446 0 nch w=1u l=180n
M3988 t1446 nw452 0 0 nch w=1u l=180n
Cnw548 nw548 0 2f
M3989 nw549 nw487 0 0 nch w=1u l=180n
M3990 nw549 nw453 0 0 nch w=1u l=180n
CT1447 t1447 0 0.1f
M3991 t1447 nw487 vdd vdd pch w=2u l=180n
M3992 nw549 nw453 t1447 vdd pch w=2u l=180n
Cnw549 nw549 0 2f
CT1448 t1448 0 0.1f
M3993 t1448 nw488 vdd vdd pch w=2u l=180n
M3994 t1448 nw454 vdd vdd pch w=2u l=180n
CT1449 t1449 0 0.1f
M3995 t1448 nw488 t1449 0 nch w=1u l=180n
M3996 t1449 nw454 0 0 nch w=1u l=180n
M3997 nw550 t1448 vdd vdd pch w=2u l=180n
M3998 nw550 t1448 0 0 nch w=1u l=180n
Cnw550 nw550 0 2f
CT1450 t1450 0 0.1f
M3999 t1450 nw489 0 0 nch w=1u l=180n
M4000 t1450 nw455 0 0 nch w=1u l=180n
CT1451 t1451 0 0.1f
M4001 t1451 nw489 vdd vdd pch w=2u l=180n
M4002 t1450 nw455 t1451 vdd pch w=2u l=180n
M4003 nw551 t1450 vdd vdd pch w=2u l=180n
M4004 nw551 t1450 0 0 nch w=1u l=180n
Cnw551 nw551 0 2f
CT1452 t1452 0 0.1f
CT1453 t1453 0 0.1f
CT1454 t1454 0 0.1f
M4005 t1452 nw490 vdd vdd pch w=2u l=180n
M4006 t1452 nw456 vdd vdd pch w=2u l=180n
CT1455 t1455 0 0.1f
M4007 t1452 nw490 t1455 0 nch w=1u l=180n
M4008 t1455 nw456 0 0 nch w=1u l=180n
M4009 t1453 nw490 vdd vdd pch w=2u l=180n
M4010 t1453 t1452 vdd vdd pch w=2u l=180n
CT1456 t1456 0 0.1f
M4011 t1453 nw490 t1456 0 nch w=1u l=180n
M4012 t1456 t1452 0 0 nch w=1u l=180n
M4013 t1454 nw456 vdd vdd pch w=2u l=180n
M4014 t1454 t1452 vdd vdd pch w=2u l=180n
CT1457 t1457 0 0.1f
M4015 t1454 nw456 t1457 0 nch w=1u l=180n
M4016 t1457 t1452 0 0 nch w=1u l=180n
M4017 nw552 t1453 vdd vdd pch w=2u l=180n
M4018 nw552 t1454 vdd vdd pch w=2u l=180n
CT1458 t1458 0 0.1f
M4019 nw552 t1453 t1458 0 nch w=1u l=180n
M4020 t1458 t1454 0 0 nch w=1u l=180n
Cnw552 nw552 0 2f
M4021 nw553 nw491 vdd vdd pch w=2u l=180n
M4022 nw553 nw457 vdd vdd pch w=2u l=180n
CT1459 t1459 0 0.1f
M4023 nw553 nw491 t1459 0 nch w=1u l=180n
M4024 t1459 nw457 0 0 nch w=1u l=180n
Cnw553 nw553 0 2f
M4025 nw554 nw492 0 0 nch w=1u l=180n
M4026 nw554 nw458 0 0 nch w=1u l=180n
CT1460 t1460 0 0.1f
M4027 t1460 nw492 vdd vdd pch w=2u l=180n
M4028 nw554 nw458 t1460 vdd pch w=2u l=180n
Cnw554 nw554 0 2f
CT1461 t1461 0 0.1f
M4029 t1461 nw493 vdd vdd pch w=2u l=180n
M4030 t1461 nw459 vdd vdd pch w=2u l=180n
CT1462 t1462 0 0.1f
M4031 t1461 nw493 t1462 0 nch w=1u l=180n
M4032 t1462 nw459 0 0 nch w=1u l=180n
M4033 nw555 t1461 vdd vdd pch w=2u l=180n
M4034 nw555 t1461 0 0 nch w=1u l=180n
Cnw555 nw555 0 2f
CT1463 t1463 0 0.1f
M4035 t1463 nw494 0 0 nch w=1u l=180n
M4036 t1463 nw460 0 0 nch w=1u l=180n
CT1464 t1464 0 0.1f
M4037 t1464 nw494 vdd vdd pch w=2u l=180n
M4038 t1463 nw460 t1464 vdd pch w=2u l=180n
M4039 nw556 t1463 vdd vdd pch w=2u l=180n
M4040 nw556 t1463 0 0 nch w=1u l=180n
Cnw556 nw556 0 2f
CT1465 t1465 0 0.1f
CT1466 t1466 0 0.1f
CT1467 t1467 0 0.1f
M4041 t1465 nw495 vdd vdd pch w=2u l=180n
M4042 t1465 nw461 vdd vdd pch w=2u l=180n
CT1468 t1468 0 0.1f
M4043 t1465 nw495 t1468 0 nch w=1u l=180n
M4044 t1468 nw461 0 0 nch w=1u l=180n
M4045 t1466 nw495 vdd vdd pch w=2u l=180n
M4046 t1466 t1465 vdd vdd pch w=2u l=180n
CT1469 t1469 0 0.1f
M4047 t1466 nw495 t1469 0 nch w=1u l=180n
M4048 t1469 t1465 0 0 nch w=1u l=180n
M4049 t1467 nw461 vdd vdd pch w=2u l=180n
M4050 t1467 t1465 vdd vdd pch w=2u l=180n
CT1470 t1470 0 0.1f
M4051 t1467 nw461 t1470 0 nch w=1u l=180n
M4052 t1470 t1465 0 0 nch w=1u l=180n
M4053 nw557 t1466 vdd vdd pch w=2u l=180n
M4054 nw557 t1467 vdd vdd pch w=2u l=180n
CT1471 t1471 0 0.1f
M4055 nw557 t1466 t1471 0 nch w=1u l=180n
M4056 t1471 t1467 0 0 nch w=1u l=180n
Cnw557 nw557 0 2f
M4057 nw558 nw496 vdd vdd pch w=2u l=180n
M4058 nw558 nw462 vdd vdd pch w=2u l=180n
CT1472 t1472 0 0.1f
M4059 nw558 nw496 t1472 0 nch w=1u l=180n
M4060 t1472 nw462 0 0 nch w=1u l=180n
Cnw558 nw558 0 2f
M4061 nw559 nw497 0 0 nch w=1u l=180n
M4062 nw559 nw463 0 0 nch w=1u l=180n
CT1473 t1473 0 0.1f
M4063 t1473 nw497 vdd vdd pch w=2u l=180n
M4064 nw559 nw463 t1473 vdd pch w=2u l=180n
Cnw559 nw559 0 2f
CT1474 t1474 0 0.1f
M4065 t1474 nw498 vdd vdd pch w=2u l=180n
M4066 t1474 nw464 vdd vdd pch w=2u l=180n
CT1475 t1475 0 0.1f
M4067 t1474 nw498 t1475 0 nch w=1u l=180n
M4068 t1475 nw464 0 0 nch w=1u l=180n
M4069 nw560 t1474 vdd vdd pch w=2u l=180n
M4070 nw560 t1474 0 0 nch w=1u l=180n
Cnw560 nw560 0 2f
CT1476 t1476 0 0.1f
M4071 t1476 nw499 0 0 nch w=1u l=180n
M4072 t1476 nw465 0 0 nch w=1u l=180n
CT1477 t1477 0 0.1f
M4073 t1477 nw499 vdd vdd pch w=2u l=180n
M4074 t1476 nw465 t1477 vdd pch w=2u l=180n
M4075 nw561 t1476 vdd vdd pch w=2u l=180n
M4076 nw561 t1476 0 0 nch w=1u l=180n
Cnw561 nw561 0 2f
CT1478 t1478 0 0.1f
CT1479 t1479 0 0.1f
CT1480 t1480 0 0.1f
M4077 t1478 nw500 vdd vdd pch w=2u l=180n
M4078 t1478 nw466 vdd vdd pch w=2u l=180n
CT1481 t1481 0 0.1f
M4079 t1478 nw500 t1481 0 nch w=1u l=180n
M4080 t1481 nw466 0 0 nch w=1u l=180n
M4081 t1479 nw500 vdd vdd pch w=2u l=180n
M4082 t1479 t1478 vdd vdd pch w=2u l=180n
CT1482 t1482 0 0.1f
M4083 t1479 nw500 t1482 0 nch w=1u l=180n
M4084 t1482 t1478 0 0 nch w=1u l=180n
M4085 t1480 nw466 vdd vdd pch w=2u l=180n
M4086 t1480 t1478 vdd vdd pch w=2u l=180n
CT1483 t1483 0 0.1f
M4087 t1480 nw466 t1483 0 nch w=1u l=180n
M4088 t1483 t1478 0 0 nch w=1u l=180n
M4089 nw562 t1479 vdd vdd pch w=2u l=180n
M4090 nw562 t1480 vdd vdd pch w=2u l=180n
CT1484 t1484 0 0.1f
M4091 nw562 t1479 t1484 0 nch w=1u l=180n
M4092 t1484 t1480 0 0 nch w=1u l=180n
Cnw562 nw562 0 2f
M4093 nw563 nw501 vdd vdd pch w=2u l=180n
M4094 nw563 nw467 vdd vdd pch w=2u l=180n
CT1485 t1485 0 0.1f
M4095 nw563 nw501 t1485 0 nch w=1u l=180n
M4096 t1485 nw467 0 0 nch w=1u l=180n
Cnw563 nw563 0 2f
M4097 nw564 nw502 0 0 nch w=1u l=180n
M4098 nw564 nw468 0 0 nch w=1u l=180n
CT1486 t1486 0 0.1f
M4099 t1486 nw502 vdd vdd pch w=2u l=180n
M4100 nw564 nw468 t1486 vdd pch w=2u l=180n
Cnw564 nw564 0 2f
CT1487 t1487 0 0.1f
M4101 t1487 nw503 vdd vdd pch w=2u l=180n
M4102 t1487 nw469 vdd vdd pch w=2u l=180n
CT1488 t1488 0 0.1f
M4103 t1487 nw503 t1488 0 nch w=1u l=180n
M4104 t1488 nw469 0 0 nch w=1u l=180n
M4105 nw565 t1487 vdd vdd pch w=2u l=180n
M4106 nw565 t1487 0 0 nch w=1u l=180n
Cnw565 nw565 0 2f
CT1489 t1489 0 0.1f
M4107 t1489 nw504 0 0 nch w=1u l=180n
M4108 t1489 nw470 0 0 nch w=1u l=180n
CT1490 t1490 0 0.1f
M4109 t1490 nw504 vdd vdd pch w=2u l=180n
M4110 t1489 nw470 t1490 vdd pch w=2u l=180n
M4111 nw566 t1489 vdd vdd pch w=2u l=180n
M4112 nw566 t1489 0 0 nch w=1u l=180n
Cnw566 nw566 0 2f
CT1491 t1491 0 0.1f
CT1492 t1492 0 0.1f
CT1493 t1493 0 0.1f
M4113 t1491 nw505 vdd vdd pch w=2u l=180n
M4114 t1491 nw471 vdd vdd pch w=2u l=180n
CT1494 t1494 0 0.1f
M4115 t1491 nw505 t1494 0 nch w=1u l=180n
M4116 t1494 nw471 0 0 nch w=1u l=180n
M4117 t1492 nw505 vdd vdd pch w=2u l=180n
M4118 t1492 t1491 vdd vdd pch w=2u l=180n
CT1495 t1495 0 0.1f
M4119 t1492 nw505 t1495 0 nch w=1u l=180n
M4120 t1495 t1491 0 0 nch w=1u l=180n
M4121 t1493 nw471 vdd vdd pch w=2u l=180n
M4122 t1493 t1491 vdd vdd pch w=2u l=180n
CT1496 t1496 0 0.1f
M4123 t1493 nw471 t1496 0 nch w=1u l=180n
M4124 t1496 t1491 0 0 nch w=1u l=180n
M4125 nw567 t1492 vdd vdd pch w=2u l=180n
M4126 nw567 t1493 vdd vdd pch w=2u l=180n
CT1497 t1497 0 0.1f
M4127 nw567 t1492 t1497 0 nch w=1u l=180n
M4128 t1497 t1493 0 0 nch w=1u l=180n
Cnw567 nw567 0 2f
M4129 nw568 nw506 vdd vdd pch w=2u l=180n
M4130 nw568 nw472 vdd vdd pch w=2u l=180n
CT1498 t1498 0 0.1f
M4131 nw568 nw506 t1498 0 nch w=1u l=180n
M4132 t1498 nw472 0 0 nch w=1u l=180n
Cnw568 nw568 0 2f
M4133 nw569 nw507 0 0 nch w=1u l=180n
M4134 nw569 nw473 0 0 nch w=1u l=180n
CT1499 t1499 0 0.1f
M4135 t1499 nw507 vdd vdd pch w=2u l=180n
M4136 nw569 nw473 t1499 vdd pch w=2u l=180n
Cnw569 nw569 0 2f
CT1500 t1500 0 0.1f
M4137 t1500 nw508 vdd vdd pch w=2u l=180n
M4138 t1500 nw474 vdd vdd pch w=2u l=180n
CT1501 t1501 0 0.1f
M4139 t1500 nw508 t1501 0 nch w=1u l=180n
M4140 t1501 nw474 0 0 nch w=1u l=180n
M4141 nw570 t1500 vdd vdd pch w=2u l=180n
M4142 nw570 t1500 0 0 nch w=1u l=180n
Cnw570 nw570 0 2f
CT1502 t1502 0 0.1f
M4143 t1502 nw509 0 0 nch w=1u l=180n
M4144 t1502 nw475 0 0 nch w=1u l=180n
CT1503 t1503 0 0.1f
M4145 t1503 nw509 vdd vdd pch w=2u l=180n
M4146 t1502 nw475 t1503 vdd pch w=2u l=180n
M4147 nw571 t1502 vdd vdd pch w=2u l=180n
M4148 nw571 t1502 0 0 nch w=1u l=180n
Cnw571 nw571 0 2f
CT1504 t1504 0 0.1f
CT1505 t1505 0 0.1f
CT1506 t1506 0 0.1f
M4149 t1504 nw510 vdd vdd pch w=2u l=180n
M4150 t1504 nw476 vdd vdd pch w=2u l=180n
CT1507 t1507 0 0.1f
M4151 t1504 nw510 t1507 0 nch w=1u l=180n
M4152 t1507 nw476 0 0 nch w=1u l=180n
M4153 t1505 nw510 vdd vdd pch w=2u l=180n
M4154 t1505 t1504 vdd vdd pch w=2u l=180n
CT1508 t1508 0 0.1f
M4155 t1505 nw510 t1508 0 nch w=1u l=180n
M4156 t1508 t1504 0 0 nch w=1u l=180n
M4157 t1506 nw476 vdd vdd pch w=2u l=180n
M4158 t1506 t1504 vdd vdd pch w=2u l=180n
CT1509 t1509 0 0.1f
M4159 t1506 nw476 t1509 0 nch w=1u l=180n
M4160 t1509 t1504 0 0 nch w=1u l=180n
M4161 nw572 t1505 vdd vdd pch w=2u l=180n
M4162 nw572 t1506 vdd vdd pch w=2u l=180n
CT1510 t1510 0 0.1f
M4163 nw572 t1505 t1510 0 nch w=1u l=180n
M4164 t1510 t1506 0 0 nch w=1u l=180n
Cnw572 nw572 0 2f
M4165 nw573 nw511 vdd vdd pch w=2u l=180n
M4166 nw573 nw477 vdd vdd pch w=2u l=180n
CT1511 t1511 0 0.1f
M4167 nw573 nw511 t1511 0 nch w=1u l=180n
M4168 t1511 nw477 0 0 nch w=1u l=180n
Cnw573 nw573 0 2f
M4169 nw574 nw512 0 0 nch w=1u l=180n
M4170 nw574 nw478 0 0 nch w=1u l=180n
CT1512 t1512 0 0.1f
M4171 t1512 nw512 vdd vdd pch w=2u l=180n
M4172 nw574 nw478 t1512 vdd pch w=2u l=180n
Cnw574 nw574 0 2f
CT1513 t1513 0 0.1f
M4173 t1513 nw513 vdd vdd pch w=2u l=180n
M4174 t1513 nw479 vdd vdd pch w=2u l=180n
CT1514 t1514 0 0.1f
M4175 t1513 nw513 t1514 0 nch w=1u l=180n
M4176 t1514 nw479 0 0 nch w=1u l=180n
M4177 nw575 t1513 vdd vdd pch w=2u l=180n
M4178 nw575 t1513 0 0 nch w=1u l=180n
Cnw575 nw575 0 2f
CT1515 t1515 0 0.1f
M4179 t1515 nw514 0 0 nch w=1u l=180n
M4180 t1515 nw480 0 0 nch w=1u l=180n
CT1516 t1516 0 0.1f
M4181 t1516 nw514 vdd vdd pch w=2u l=180n
M4182 t1515 nw480 t1516 vdd pch w=2u l=180n
M4183 nw576 t1515 vdd vdd pch w=2u l=180n
M4184 nw576 t1515 0 0 nch w=1u l=180n
Cnw576 nw576 0 2f
CT1517 t1517 0 0.1f
CT1518 t1518 0 0.1f
CT1519 t1519 0 0.1f
M4185 t1517 nw515 vdd vdd pch w=2u l=180n
M4186 t1517 nw481 vdd vdd pch w=2u l=180n
CT1520 t1520 0 0.1f
M4187 t1517 nw515 t1520 0 nch w=1u l=180n
M4188 t1520 nw481 0 0 nch w=1u l=180n
M4189 t1518 nw515 vdd vdd pch w=2u l=180n
M4190 t1518 t1517 vdd vdd pch w=2u l=180n
CT1521 t1521 0 0.1f
M4191 t1518 nw515 t1521 0 nch w=1u l=180n
M4192 t1521 t1517 0 0 nch w=1u l=180n
M4193 t1519 nw481 vdd vdd pch w=2u l=180n
M4194 t1519 t1517 vdd vdd pch w=2u l=180n
CT1522 t1522 0 0.1f
M4195 t1519 nw481 t1522 0 nch w=1u l=180n
M4196 t1522 t1517 0 0 nch w=1u l=180n
M4197 nw577 t1518 vdd vdd pch w=2u l=180n
M4198 nw577 t1519 vdd vdd pch w=2u l=180n
CT1523 t1523 0 0.1f
M4199 nw577 t1518 t1523 0 nch w=1u l=180n
M4200 t1523 t1519 0 0 nch w=1u l=180n
Cnw577 nw577 0 2f
M4201 nw578 nw516 vdd vdd pch w=2u l=180n
M4202 nw578 nw482 vdd vdd pch w=2u l=180n
CT1524 t1524 0 0.1f
M4203 nw578 nw516 t1524 0 nch w=1u l=180n
M4204 t1524 nw482 0 0 nch w=1u l=180n
Cnw578 nw578 0 2f
M4205 nw579 nw517 0 0 nch w=1u l=180n
M4206 nw579 nw483 0 0 nch w=1u l=180n
CT1525 t1525 0 0.1f
M4207 t1525 nw517 vdd vdd pch w=2u l=180n
M4208 nw579 nw483 t1525 vdd pch w=2u l=180n
Cnw579 nw579 0 2f
CT1526 t1526 0 0.1f
M4209 t1526 nw518 vdd vdd pch w=2u l=180n
M4210 t1526 nw484 vdd vdd pch w=2u l=180n
CT1527 t1527 0 0.1f
M4211 t1526 nw518 t1527 0 nch w=1u l=180n
M4212 t1527 nw484 0 0 nch w=1u l=180n
M4213 nw580 t1526 vdd vdd pch w=2u l=180n
M4214 nw580 t1526 0 0 nch w=1u l=180n
Cnw580 nw580 0 2f
CT1528 t1528 0 0.1f
M4215 t1528 nw519 0 0 nch w=1u l=180n
M4216 t1528 nw485 0 0 nch w=1u l=180n
CT1529 t1529 0 0.1f
M4217 t1529 nw519 vdd vdd pch w=2u l=180n
M4218 t1528 nw485 t1529 vdd pch w=2u l=180n
M4219 nw581 t1528 vdd vdd pch w=2u l=180n
M4220 nw581 t1528 0 0 nch w=1u l=180n
Cnw581 nw581 0 2f
CT1530 t1530 0 0.1f
CT1531 t1531 0 0.1f
CT1532 t1532 0 0.1f
M4221 t1530 nw520 vdd vdd pch w=2u l=180n
M4222 t1530 nw486 vdd vdd pch w=2u l=180n
CT1533 t1533 0 0.1f
M4223 t1530 nw520 t1533 0 nch w=1u l=180n
M4224 t1533 nw486 0 0 nch w=1u l=180n
M4225 t1531 nw520 vdd vdd pch w=2u l=180n
M4226 t1531 t1530 vdd vdd pch w=2u l=180n
CT1534 t1534 0 0.1f
M4227 t1531 nw520 t1534 0 nch w=1u l=180n
M4228 t1534 t1530 0 0 nch w=1u l=180n
M4229 t1532 nw486 vdd vdd pch w=2u l=180n
M4230 t1532 t1530 vdd vdd pch w=2u l=180n
CT1535 t1535 0 0.1f
M4231 t1532 nw486 t1535 0 nch w=1u l=180n
M4232 t1535 t1530 0 0 nch w=1u l=180n
M4233 nw582 t1531 vdd vdd pch w=2u l=180n
M4234 nw582 t1532 vdd vdd pch w=2u l=180n
CT1536 t1536 0 0.1f
M4235 nw582 t1531 t1536 0 nch w=1u l=180n
M4236 t1536 t1532 0 0 nch w=1u l=180n
Cnw582 nw582 0 2f
M4237 nw583 nw521 vdd vdd pch w=2u l=180n
M4238 nw583 nw487 vdd vdd pch w=2u l=180n
CT1537 t1537 0 0.1f
M4239 nw583 nw521 t1537 0 nch w=1u l=180n
M4240 t1537 nw487 0 0 nch w=1u l=180n
Cnw583 nw583 0 2f
M4241 nw584 nw522 0 0 nch w=1u l=180n
M4242 nw584 nw488 0 0 nch w=1u l=180n
CT1538 t1538 0 0.1f
M4243 t1538 nw522 vdd vdd pch w=2u l=180n
M4244 nw584 nw488 t1538 vdd pch w=2u l=180n
Cnw584 nw584 0 2f
CT1539 t1539 0 0.1f
M4245 t1539 nw523 vdd vdd pch w=2u l=180n
M4246 t1539 nw489 vdd vdd pch w=2u l=180n
CT1540 t1540 0 0.1f
M4247 t1539 nw523 t1540 0 nch w=1u l=180n
M4248 t1540 nw489 0 0 nch w=1u l=180n
M4249 nw585 t1539 vdd vdd pch w=2u l=180n
M4250 nw585 t1539 0 0 nch w=1u l=180n
Cnw585 nw585 0 2f
CT1541 t1541 0 0.1f
M4251 t1541 nw524 0 0 nch w=1u l=180n
M4252 t1541 nw490 0 0 nch w=1u l=180n
CT1542 t1542 0 0.1f
M4253 t1542 nw524 vdd vdd pch w=2u l=180n
M4254 t1541 nw490 t1542 vdd pch w=2u l=180n
M4255 nw586 t1541 vdd vdd pch w=2u l=180n
M4256 nw586 t1541 0 0 nch w=1u l=180n
Cnw586 nw586 0 2f
CT1543 t1543 0 0.1f
CT1544 t1544 0 0.1f
CT1545 t1545 0 0.1f
M4257 t1543 nw525 vdd vdd pch w=2u l=180n
M4258 t1543 nw491 vdd vdd pch w=2u l=180n
CT1546 t1546 0 0.1f
M4259 t1543 nw525 t1546 0 nch w=1u l=180n
M4260 t1546 nw491 0 0 nch w=1u l=180n
M4261 t1544 nw525 vdd vdd pch w=2u l=180n
M4262 t1544 t1543 vdd vdd pch w=2u l=180n
CT1547 t1547 0 0.1f
M4263 t1544 nw525 t1547 0 nch w=1u l=180n
M4264 t1547 t1543 0 0 nch w=1u l=180n
M4265 t1545 nw491 vdd vdd pch w=2u l=180n
M4266 t1545 t1543 vdd vdd pch w=2u l=180n
CT1548 t1548 0 0.1f
M4267 t1545 nw491 t1548 0 nch w=1u l=180n
M4268 t1548 t1543 0 0 nch w=1u l=180n
M4269 nw587 t1544 vdd vdd pch w=2u l=180n
M4270 nw587 t1545 vdd vdd pch w=2u l=180n
CT1549 t1549 0 0.1f
M4271 nw587 t1544 t1549 0 nch w=1u l=180n
M4272 t1549 t1545 0 0 nch w=1u l=180n
Cnw587 nw587 0 2f
M4273 nw588 nw526 vdd vdd pch w=2u l=180n
M4274 nw588 nw492 vdd vdd pch w=2u l=180n
CT1550 t1550 0 0.1f
M4275 nw588 nw526 t1550 0 nch w=1u l=180n
M4276 t1550 nw492 0 0 nch w=1u l=180n
Cnw588 nw588 0 2f
M4277 nw589 nw527 0 0 nch w=1u l=180n
M4278 nw589 nw493 0 0 nch w=1u l=180n
CT1551 t1551 0 0.1f
M4279 t1551 nw527 vdd vdd pch w=2u l=180n
M4280 nw589 nw493 t1551 vdd pch w=2u l=180n
Cnw589 nw589 0 2f
CT1552 t1552 0 0.1f
M4281 t1552 nw528 vdd vdd pch w=2u l=180n
M4282 t1552 nw494 vdd vdd pch w=2u l=180n
CT1553 t1553 0 0.1f
M4283 t1552 nw528 t1553 0 nch w=1u l=180n
M4284 t1553 nw494 0 0 nch w=1u l=180n
M4285 nw590 t1552 vdd vdd pch w=2u l=180n
M4286 nw590 t1552 0 0 nch w=1u l=180n
Cnw590 nw590 0 2f
CT1554 t1554 0 0.1f
M4287 t1554 nw529 0 0 nch w=1u l=180n
M4288 t1554 nw495 0 0 nch w=1u l=180n
CT1555 t1555 0 0.1f
M4289 t1555 nw529 vdd vdd pch w=2u l=180n
M4290 t1554 nw495 t1555 vdd pch w=2u l=180n
M4291 nw591 t1554 vdd vdd pch w=2u l=180n
M4292 nw591 t1554 0 0 nch w=1u l=180n
Cnw591 nw591 0 2f
CT1556 t1556 0 0.1f
CT1557 t1557 0 0.1f
CT1558 t1558 0 0.1f
M4293 t1556 nw530 vdd vdd pch w=2u l=180n
M4294 t1556 nw496 vdd vdd pch w=2u l=180n
CT1559 t1559 0 0.1f
M4295 t1556 nw530 t1559 0 nch w=1u l=180n
M4296 t1559 nw496 0 0 nch w=1u l=180n
M4297 t1557 nw530 vdd vdd pch w=2u l=180n
M4298 t1557 t1556 vdd vdd pch w=2u l=180n
CT1560 t1560 0 0.1f
M4299 t1557 nw530 t1560 0 nch w=1u l=180n
M4300 t1560 t1556 0 0 nch w=1u l=180n
M4301 t1558 nw496 vdd vdd pch w=2u l=180n
M4302 t1558 t1556 vdd vdd pch w=2u l=180n
CT1561 t1561 0 0.1f
M4303 t1558 nw496 t1561 0 nch w=1u l=180n
M4304 t1561 t1556 0 0 nch w=1u l=180n
M4305 nw592 t1557 vdd vdd pch w=2u l=180n
M4306 nw592 t1558 vdd vdd pch w=2u l=180n
CT1562 t1562 0 0.1f
M4307 nw592 t1557 t1562 0 nch w=1u l=180n
M4308 t1562 t1558 0 0 nch w=1u l=180n
Cnw592 nw592 0 2f
M4309 nw593 nw531 vdd vdd pch w=2u l=180n
M4310 nw593 nw497 vdd vdd pch w=2u l=180n
CT1563 t1563 0 0.1f
M4311 nw593 nw531 t1563 0 nch w=1u l=180n
M4312 t1563 nw497 0 0 nch w=1u l=180n
Cnw593 nw593 0 2f
M4313 nw594 nw532 0 0 nch w=1u l=180n
M4314 nw594 nw498 0 0 nch w=1u l=180n
CT1564 t1564 0 0.1f
M4315 t1564 nw532 vdd vdd pch w=2u l=180n
M4316 nw594 nw498 t1564 vdd pch w=2u l=180n
Cnw594 nw594 0 2f
CT1565 t1565 0 0.1f
M4317 t1565 nw533 vdd vdd pch w=2u l=180n
M4318 t1565 nw499 vdd vdd pch w=2u l=180n
CT1566 t1566 0 0.1f
M4319 t1565 nw533 t1566 0 nch w=1u l=180n
M4320 t1566 nw499 0 0 nch w=1u l=180n
M4321 nw595 t1565 vdd vdd pch w=2u l=180n
M4322 nw595 t1565 0 0 nch w=1u l=180n
Cnw595 nw595 0 2f
CT1567 t1567 0 0.1f
M4323 t1567 nw534 0 0 nch w=1u l=180n
M4324 t1567 nw500 0 0 nch w=1u l=180n
CT1568 t1568 0 0.1f
M4325 t1568 nw534 vdd vdd pch w=2u l=180n
M4326 t1567 nw500 t1568 vdd pch w=2u l=180n
M4327 nw596 t1567 vdd vdd pch w=2u l=180n
M4328 nw596 t1567 0 0 nch w=1u l=180n
Cnw596 nw596 0 2f
CT1569 t1569 0 0.1f
CT1570 t1570 0 0.1f
CT1571 t1571 0 0.1f
M4329 t1569 nw535 vdd vdd pch w=2u l=180n
M4330 t1569 nw501 vdd vdd pch w=2u l=180n
CT1572 t1572 0 0.1f
M4331 t1569 nw535 t1572 0 nch w=1u l=180n
M4332 t1572 nw501 0 0 nch w=1u l=180n
M4333 t1570 nw535 vdd vdd pch w=2u l=180n
M4334 t1570 t1569 vdd vdd pch w=2u l=180n
CT1573 t1573 0 0.1f
M4335 t1570 nw535 t1573 0 nch w=1u l=180n
M4336 t1573 t1569 0 0 nch w=1u l=180n
M4337 t1571 nw501 vdd vdd pch w=2u l=180n
M4338 t1571 t1569 vdd vdd pch w=2u l=180n
CT1574 t1574 0 0.1f
M4339 t1571 nw501 t1574 0 nch w=1u l=180n
M4340 t1574 t1569 0 0 nch w=1u l=180n
M4341 nw597 t1570 vdd vdd pch w=2u l=180n
M4342 nw597 t1571 vdd vdd pch w=2u l=180n
CT1575 t1575 0 0.1f
M4343 nw597 t1570 t1575 0 nch w=1u l=180n
M4344 t1575 t1571 0 0 nch w=1u l=180n
Cnw597 nw597 0 2f
M4345 nw598 nw536 vdd vdd pch w=2u l=180n
M4346 nw598 nw502 vdd vdd pch w=2u l=180n
CT1576 t1576 0 0.1f
M4347 nw598 nw536 t1576 0 nch w=1u l=180n
M4348 t1576 nw502 0 0 nch w=1u l=180n
Cnw598 nw598 0 2f
M4349 nw599 nw537 0 0 nch w=1u l=180n
M4350 nw599 nw503 0 0 nch w=1u l=180n
CT1577 t1577 0 0.1f
M4351 t1577 nw537 vdd vdd pch w=2u l=180n
M4352 nw599 nw503 t1577 vdd pch w=2u l=180n
Cnw599 nw599 0 2f
CT1578 t1578 0 0.1f
M4353 t1578 nw538 vdd vdd pch w=2u l=180n
M4354 t1578 nw504 vdd vdd pch w=2u l=180n
CT1579 t1579 0 0.1f
M4355 t1578 nw538 t1579 0 nch w=1u l=180n
M4356 t1579 nw504 0 0 nch w=1u l=180n
M4357 nw600 t1578 vdd vdd pch w=2u l=180n
M4358 nw600 t1578 0 0 nch w=1u l=180n
Cnw600 nw600 0 2f
CT1580 t1580 0 0.1f
M4359 t1580 nw539 0 0 nch w=1u l=180n
M4360 t1580 nw505 0 0 nch w=1u l=180n
CT1581 t1581 0 0.1f
M4361 t1581 nw539 vdd vdd pch w=2u l=180n
M4362 t1580 nw505 t1581 vdd pch w=2u l=180n
M4363 nw601 t1580 vdd vdd pch w=2u l=180n
M4364 nw601 t1580 0 0 nch w=1u l=180n
Cnw601 nw601 0 2f
CT1582 t1582 0 0.1f
CT1583 t1583 0 0.1f
CT1584 t1584 0 0.1f
M4365 t1582 nw540 vdd vdd pch w=2u l=180n
M4366 t1582 nw506 vdd vdd pch w=2u l=180n
CT1585 t1585 0 0.1f
M4367 t1582 nw540 t1585 0 nch w=1u l=180n
M4368 t1585 nw506 0 0 nch w=1u l=180n
M4369 t1583 nw540 vdd vdd pch w=2u l=180n
M4370 t1583 t1582 vdd vdd pch w=2u l=180n
CT1586 t1586 0 0.1f
M4371 t1583 nw540 t1586 0 nch w=1u l=180n
M4372 t1586 t1582 0 0 nch w=1u l=180n
M4373 t1584 nw506 vdd vdd pch w=2u l=180n
M4374 t1584 t1582 vdd vdd pch w=2u l=180n
CT1587 t1587 0 0.1f
M4375 t1584 nw506 t1587 0 nch w=1u l=180n
M4376 t1587 t1582 0 0 nch w=1u l=180n
M4377 nw602 t1583 vdd vdd pch w=2u l=180n
M4378 nw602 t1584 vdd vdd pch w=2u l=180n
CT1588 t1588 0 0.1f
M4379 nw602 t1583 t1588 0 nch w=1u l=180n
M4380 t1588 t1584 0 0 nch w=1u l=180n
Cnw602 nw602 0 2f
M4381 nw603 nw541 vdd vdd pch w=2u l=180n
M4382 nw603 nw507 vdd vdd pch w=2u l=180n
CT1589 t1589 0 0.1f
M4383 nw603 nw541 t1589 0 nch w=1u l=180n
M4384 t1589 nw507 0 0 nch w=1u l=180n
Cnw603 nw603 0 2f
M4385 nw604 nw542 0 0 nch w=1u l=180n
M4386 nw604 nw508 0 0 nch w=1u l=180n
CT1590 t1590 0 0.1f
M4387 t1590 nw542 vdd vdd pch w=2u l=180n
M4388 nw604 nw508 t1590 vdd pch w=2u l=180n
Cnw604 nw604 0 2f
CT1591 t1591 0 0.1f
M4389 t1591 nw543 vdd vdd pch w=2u l=180n
M4390 t1591 nw509 vdd vdd pch w=2u l=180n
CT1592 t1592 0 0.1f
M4391 t1591 nw543 t1592 0 nch w=1u l=180n
M4392 t1592 nw509 0 0 nch w=1u l=180n
M4393 nw605 t1591 vdd vdd pch w=2u l=180n
M4394 nw605 t1591 0 0 nch w=1u l=180n
Cnw605 nw605 0 2f
CT1593 t1593 0 0.1f
M4395 t1593 nw544 0 0 nch w=1u l=180n
M4396 t1593 nw510 0 0 nch w=1u l=180n
CT1594 t1594 0 0.1f
M4397 t1594 nw544 vdd vdd pch w=2u l=180n
M4398 t1593 nw510 t1594 vdd pch w=2u l=180n
M4399 nw606 t1593 vdd vdd pch w=2u l=180n
M4400 nw606 t1593 0 0 nch w=1u l=180n
Cnw606 nw606 0 2f
CT1595 t1595 0 0.1f
CT1596 t1596 0 0.1f
CT1597 t1597 0 0.1f
M4401 t1595 nw545 vdd vdd pch w=2u l=180n
M4402 t1595 nw511 vdd vdd pch w=2u l=180n
CT1598 t1598 0 0.1f
M4403 t1595 nw545 t1598 0 nch w=1u l=180n
M4404 t1598 nw511 0 0 nch w=1u l=180n
M4405 t1596 nw545 vdd vdd pch w=2u l=180n
M4406 t1596 t1595 vdd vdd pch w=2u l=180n
CT1599 t1599 0 0.1f
M4407 t1596 nw545 t1599 0 nch w=1u l=180n
M4408 t1599 t1595 0 0 nch w=1u l=180n
M4409 t1597 nw511 vdd vdd pch w=2u l=180n
M4410 t1597 t1595 vdd vdd pch w=2u l=180n
CT1600 t1600 0 0.1f
M4411 t1597 nw511 t1600 0 nch w=1u l=180n
M4412 t1600 t1595 0 0 nch w=1u l=180n
M4413 nw607 t1596 vdd vdd pch w=2u l=180n
M4414 nw607 t1597 vdd vdd pch w=2u l=180n
CT1601 t1601 0 0.1f
M4415 nw607 t1596 t1601 0 nch w=1u l=180n
M4416 t1601 t1597 0 0 nch w=1u l=180n
Cnw607 nw607 0 2f
M4417 nw608 nw546 vdd vdd pch w=2u l=180n
M4418 nw608 nw512 vdd vdd pch w=2u l=180n
CT1602 t1602 0 0.1f
M4419 nw608 nw546 t1602 0 nch w=1u l=180n
M4420 t1602 nw512 0 0 nch w=1u l=180n
Cnw608 nw608 0 2f
M4421 nw609 nw547 0 0 nch w=1u l=180n
M4422 nw609 nw513 0 0 nch w=1u l=180n
CT1603 t1603 0 0.1f
M4423 t1603 nw547 vdd vdd pch w=2u l=180n
M4424 nw609 nw513 t1603 vdd pch w=2u l=180n
Cnw609 nw609 0 2f
CT1604 t1604 0 0.1f
M4425 t1604 nw548 vdd vdd pch w=2u l=180n
M4426 t1604 nw514 vdd vdd pch w=2u l=180n
CT1605 t1605 0 0.1f
M4427 t1604 nw548 t1605 0 nch w=1u l=180n
M4428 t1605 nw514 0 0 nch w=1u l=180n
M4429 nw610 t1604 vdd vdd pch w=2u l=180n
M4430 nw610 t1604 0 0 nch w=1u l=180n
Cnw610 nw610 0 2f
CT1606 t1606 0 0.1f
M4431 t1606 nw549 0 0 nch w=1u l=180n
M4432 t1606 nw515 0 0 nch w=1u l=180n
CT1607 t1607 0 0.1f
M4433 t1607 nw549 vdd vdd pch w=2u l=180n
M4434 t1606 nw515 t1607 vdd pch w=2u l=180n
M4435 nw611 t1606 vdd vdd pch w=2u l=180n
M4436 nw611 t1606 0 0 nch w=1u l=180n
Cnw611 nw611 0 2f
CT1608 t1608 0 0.1f
CT1609 t1609 0 0.1f
CT1610 t1610 0 0.1f
M4437 t1608 nw550 vdd vdd pch w=2u l=180n
M4438 t1608 nw516 vdd vdd pch w=2u l=180n
CT1611 t1611 0 0.1f
M4439 t1608 nw550 t1611 0 nch w=1u l=180n
M4440 t1611 nw516 0 0 nch w=1u l=180n
M4441 t1609 nw550 vdd vdd pch w=2u l=180n
M4442 t1609 t1608 vdd vdd pch w=2u l=180n
CT1612 t1612 0 0.1f
M4443 t1609 nw550 t1612 0 nch w=1u l=180n
M4444 t1612 t1608 0 0 nch w=1u l=180n
M4445 t1610 nw516 vdd vdd pch w=2u l=180n
M4446 t1610 t1608 vdd vdd pch w=2u l=180n
CT1613 t1613 0 0.1f
M4447 t1610 nw516 t1613 0 nch w=1u l=180n
M4448 t1613 t1608 0 0 nch w=1u l=180n
M4449 nw612 t1609 vdd vdd pch w=2u l=180n
M4450 nw612 t1610 vdd vdd pch w=2u l=180n
CT1614 t1614 0 0.1f
M4451 nw612 t1609 t1614 0 nch w=1u l=180n
M4452 t1614 t1610 0 0 nch w=1u l=180n
Cnw612 nw612 0 2f
M4453 nw613 nw551 vdd vdd pch w=2u l=180n
M4454 nw613 nw517 vdd vdd pch w=2u l=180n
CT1615 t1615 0 0.1f
M4455 nw613 nw551 t1615 0 nch w=1u l=180n
M4456 t1615 nw517 0 0 nch w=1u l=180n
Cnw613 nw613 0 2f
M4457 nw614 nw552 0 0 nch w=1u l=180n
M4458 nw614 nw518 0 0 nch w=1u l=180n
CT1616 t1616 0 0.1f
M4459 t1616 nw552 vdd vdd pch w=2u l=180n
M4460 nw614 nw518 t1616 vdd pch w=2u l=180n
Cnw614 nw614 0 2f
CT1617 t1617 0 0.1f
M4461 t1617 nw553 vdd vdd pch w=2u l=180n
M4462 t1617 nw519 vdd vdd pch w=2u l=180n
CT1618 t1618 0 0.1f
M4463 t1617 nw553 t1618 0 nch w=1u l=180n
M4464 t1618 nw519 0 0 nch w=1u l=180n
M4465 nw615 t1617 vdd vdd pch w=2u l=180n
M4466 nw615 t1617 0 0 nch w=1u l=180n
Cnw615 nw615 0 2f
CT1619 t1619 0 0.1f
M4467 t1619 nw554 0 0 nch w=1u l=180n
M4468 t1619 nw520 0 0 nch w=1u l=180n
CT1620 t1620 0 0.1f
M4469 t1620 nw554 vdd vdd pch w=2u l=180n
M4470 t1619 nw520 t1620 vdd pch w=2u l=180n
M4471 nw616 t1619 vdd vdd pch w=2u l=180n
M4472 nw616 t1619 0 0 nch w=1u l=180n
Cnw616 nw616 0 2f
CT1621 t1621 0 0.1f
CT1622 t1622 0 0.1f
CT1623 t1623 0 0.1f
M4473 t1621 nw555 vdd vdd pch w=2u l=180n
M4474 t1621 nw521 vdd vdd pch w=2u l=180n
CT1624 t1624 0 0.1f
M4475 t1621 nw555 t1624 0 nch w=1u l=180n
M4476 t1624 nw521 0 0 nch w=1u l=180n
M4477 t1622 nw555 vdd vdd pch w=2u l=180n
M4478 t1622 t1621 vdd vdd pch w=2u l=180n
CT1625 t1625 0 0.1f
M4479 t1622 nw555 t1625 0 nch w=1u l=180n
M4480 t1625 t1621 0 0 nch w=1u l=180n
M4481 t1623 nw521 vdd vdd pch w=2u l=180n
M4482 t1623 t1621 vdd vdd pch w=2u l=180n
CT1626 t1626 0 0.1f
M4483 t1623 nw521 t1626 0 nch w=1u l=180n
M4484 t1626 t1621 0 0 nch w=1u l=180n
M4485 nw617 t1622 vdd vdd pch w=2u l=180n
M4486 nw617 t1623 vdd vdd pch w=2u l=180n
CT1627 t1627 0 0.1f
M4487 nw617 t1622 t1627 0 nch w=1u l=180n
M4488 t1627 t1623 0 0 nch w=1u l=180n
Cnw617 nw617 0 2f
M4489 nw618 nw556 vdd vdd pch w=2u l=180n
M4490 nw618 nw522 vdd vdd pch w=2u l=180n
CT1628 t1628 0 0.1f
M4491 nw618 nw556 t1628 0 nch w=1u l=180n
M4492 t1628 nw522 0 0 nch w=1u l=180n
Cnw618 nw618 0 2f
M4493 nw619 nw557 0 0 nch w=1u l=180n
M4494 nw619 nw523 0 0 nch w=1u l=180n
CT1629 t1629 0 0.1f
M4495 t1629 nw557 vdd vdd pch w=2u l=180n
M4496 nw619 nw523 t1629 vdd pch w=2u l=180n
Cnw619 nw619 0 2f
CT1630 t1630 0 0.1f
M4497 t1630 nw558 vdd vdd pch w=2u l=180n
M4498 t1630 nw524 vdd vdd pch w=2u l=180n
CT1631 t1631 0 0.1f
M4499 t1630 nw558 t1631 0 nch w=1u l=180n
M4500 t1631 nw524 0 0 nch w=1u l=180n
M4501 nw620 t1630 vdd vdd pch w=2u l=180n
M4502 nw620 t1630 0 0 nch w=1u l=180n
Cnw620 nw620 0 2f
CT1632 t1632 0 0.1f
M4503 t1632 nw559 0 0 nch w=1u l=180n
M4504 t1632 nw525 0 0 nch w=1u l=180n
CT1633 t1633 0 0.1f
M4505 t1633 nw559 vdd vdd pch w=2u l=180n
M4506 t1632 nw525 t1633 vdd pch w=2u l=180n
M4507 nw621 t1632 vdd vdd pch w=2u l=180n
M4508 nw621 t1632 0 0 nch w=1u l=180n
Cnw621 nw621 0 2f
CT1634 t1634 0 0.1f
CT1635 t1635 0 0.1f
CT1636 t1636 0 0.1f
M4509 t1634 nw560 vdd vdd pch w=2u l=180n
M4510 t1634 nw526 vdd vdd pch w=2u l=180n
CT1637 t1637 0 0.1f
M4511 t1634 nw560 t1637 0 nch w=1u l=180n
M4512 t1637 nw526 0 0 nch w=1u l=180n
M4513 t1635 nw560 vdd vdd pch w=2u l=180n
M4514 t1635 t1634 vdd vdd pch w=2u l=180n
CT1638 t1638 0 0.1f
M4515 t1635 nw560 t1638 0 nch w=1u l=180n
M4516 t1638 t1634 0 0 nch w=1u l=180n
M4517 t1636 nw526 vdd vdd pch w=2u l=180n
M4518 t1636 t1634 vdd vdd pch w=2u l=180n
CT1639 t1639 0 0.1f
M4519 t1636 nw526 t1639 0 nch w=1u l=180n
M4520 t1639 t1634 0 0 nch w=1u l=180n
M4521 nw622 t1635 vdd vdd pch w=2u l=180n
M4522 nw622 t1636 vdd vdd pch w=2u l=180n
CT1640 t1640 0 0.1f
M4523 nw622 t1635 t1640 0 nch w=1u l=180n
M4524 t1640 t1636 0 0 nch w=1u l=180n
Cnw622 nw622 0 2f
M4525 nw623 nw561 vdd vdd pch w=2u l=180n
M4526 nw623 nw527 vdd vdd pch w=2u l=180n
CT1641 t1641 0 0.1f
M4527 nw623 nw561 t1641 0 nch w=1u l=180n
M4528 t1641 nw527 0 0 nch w=1u l=180n
Cnw623 nw623 0 2f
M4529 nw624 nw562 0 0 nch w=1u l=180n
M4530 nw624 nw528 0 0 nch w=1u l=180n
CT1642 t1642 0 0.1f
M4531 t1642 nw562 vdd vdd pch w=2u l=180n
M4532 nw624 nw528 t1642 vdd pch w=2u l=180n
Cnw624 nw624 0 2f
CT1643 t1643 0 0.1f
M4533 t1643 nw563 vdd vdd pch w=2u l=180n
M4534 t1643 nw529 vdd vdd pch w=2u l=180n
CT1644 t1644 0 0.1f
M4535 t1643 nw563 t1644 0 nch w=1u l=180n
M4536 t1644 nw529 0 0 nch w=1u l=180n
M4537 nw625 t1643 vdd vdd pch w=2u l=180n
M4538 nw625 t1643 0 0 nch w=1u l=180n
Cnw625 nw625 0 2f
CT1645 t1645 0 0.1f
M4539 t1645 nw564 0 0 nch w=1u l=180n
M4540 t1645 nw530 0 0 nch w=1u l=180n
CT1646 t1646 0 0.1f
M4541 t1646 nw564 vdd vdd pch w=2u l=180n
M4542 t1645 nw530 t1646 vdd pch w=2u l=180n
M4543 nw626 t1645 vdd vdd pch w=2u l=180n
M4544 nw626 t1645 0 0 nch w=1u l=180n
Cnw626 nw626 0 2f
CT1647 t1647 0 0.1f
CT1648 t1648 0 0.1f
CT1649 t1649 0 0.1f
M4545 t1647 nw565 vdd vdd pch w=2u l=180n
M4546 t1647 nw531 vdd vdd pch w=2u l=180n
CT1650 t1650 0 0.1f
M4547 t1647 nw565 t1650 0 nch w=1u l=180n
M4548 t1650 nw531 0 0 nch w=1u l=180n
M4549 t1648 nw565 vdd vdd pch w=2u l=180n
M4550 t1648 t1647 vdd vdd pch w=2u l=180n
CT1651 t1651 0 0.1f
M4551 t1648 nw565 t1651 0 nch w=1u l=180n
M4552 t1651 t1647 0 0 nch w=1u l=180n
M4553 t1649 nw531 vdd vdd pch w=2u l=180n
M4554 t1649 t1647 vdd vdd pch w=2u l=180n
CT1652 t1652 0 0.1f
M4555 t1649 nw531 t1652 0 nch w=1u l=180n
M4556 t1652 t1647 0 0 nch w=1u l=180n
M4557 nw627 t1648 vdd vdd pch w=2u l=180n
M4558 nw627 t1649 vdd vdd pch w=2u l=180n
CT1653 t1653 0 0.1f
M4559 nw627 t1648 t1653 0 nch w=1u l=180n
M4560 t1653 t1649 0 0 nch w=1u l=180n
Cnw627 nw627 0 2f
M4561 nw628 nw566 vdd vdd pch w=2u l=180n
M4562 nw628 nw532 vdd vdd pch w=2u l=180n
CT1654 t1654 0 0.1f
M4563 nw628 nw566 t1654 0 nch w=1u l=180n
M4564 t1654 nw532 0 0 nch w=1u l=180n
Cnw628 nw628 0 2f
M4565 nw629 nw567 0 0 nch w=1u l=180n
M4566 nw629 nw533 0 0 nch w=1u l=180n
CT1655 t1655 0 0.1f
M4567 t1655 nw567 vdd vdd pch w=2u l=180n
M4568 nw629 nw533 t1655 vdd pch w=2u l=180n
Cnw629 nw629 0 2f
CT1656 t1656 0 0.1f
M4569 t1656 nw568 vdd vdd pch w=2u l=180n
M4570 t1656 nw534 vdd vdd pch w=2u l=180n
CT1657 t1657 0 0.1f
M4571 t1656 nw568 t1657 0 nch w=1u l=180n
M4572 t1657 nw534 0 0 nch w=1u l=180n
M4573 nw630 t1656 vdd vdd pch w=2u l=180n
M4574 nw630 t1656 0 0 nch w=1u l=180n
Cnw630 nw630 0 2f
CT1658 t1658 0 0.1f
M4575 t1658 nw569 0 0 nch w=1u l=180n
M4576 t1658 nw535 0 0 nch w=1u l=180n
CT1659 t1659 0 0.1f
M4577 t1659 nw569 vdd vdd pch w=2u l=180n
M4578 t1658 nw535 t1659 vdd pch w=2u l=180n
M4579 nw631 t1658 vdd vdd pch w=2u l=180n
M4580 nw631 t1658 0 0 nch w=1u l=180n
Cnw631 nw631 0 2f
CT1660 t1660 0 0.1f
CT1661 t1661 0 0.1f
CT1662 t1662 0 0.1f
M4581 t1660 nw570 vdd vdd pch w=2u l=180n
M4582 t1660 nw536 vdd vdd pch w=2u l=180n
CT1663 t1663 0 0.1f
M4583 t1660 nw570 t1663 0 nch w=1u l=180n
M4584 t1663 nw536 0 0 nch w=1u l=180n
M4585 t1661 nw570 vdd vdd pch w=2u l=180n
M4586 t1661 t1660 vdd vdd pch w=2u l=180n
CT1664 t1664 0 0.1f
M4587 t1661 nw570 t1664 0 nch w=1u l=180n
M4588 t1664 t1660 0 0 nch w=1u l=180n
M4589 t1662 nw536 vdd vdd pch w=2u l=180n
M4590 t1662 t1660 vdd vdd pch w=2u l=180n
CT1665 t1665 0 0.1f
M4591 t1662 nw536 t1665 0 nch w=1u l=180n
M4592 t1665 t1660 0 0 nch w=1u l=180n
M4593 nw632 t1661 vdd vdd pch w=2u l=180n
M4594 nw632 t1662 vdd vdd pch w=2u l=180n
CT1666 t1666 0 0.1f
M4595 nw632 t1661 t1666 0 nch w=1u l=180n
M4596 t1666 t1662 0 0 nch w=1u l=180n
Cnw632 nw632 0 2f
M4597 nw633 nw571 vdd vdd pch w=2u l=180n
M4598 nw633 nw537 vdd vdd pch w=2u l=180n
CT1667 t1667 0 0.1f
M4599 nw633 nw571 t1667 0 nch w=1u l=180n
M4600 t1667 nw537 0 0 nch w=1u l=180n
Cnw633 nw633 0 2f
M4601 nw634 nw572 0 0 nch w=1u l=180n
M4602 nw634 nw538 0 0 nch w=1u l=180n
CT1668 t1668 0 0.1f
M4603 t1668 nw572 vdd vdd pch w=2u l=180n
M4604 nw634 nw538 t1668 vdd pch w=2u l=180n
Cnw634 nw634 0 2f
CT1669 t1669 0 0.1f
M4605 t1669 nw573 vdd vdd pch w=2u l=180n
M4606 t1669 nw539 vdd vdd pch w=2u l=180n
CT1670 t1670 0 0.1f
M4607 t1669 nw573 t1670 0 nch w=1u l=180n
M4608 t1670 nw539 0 0 nch w=1u l=180n
M4609 nw635 t1669 vdd vdd pch w=2u l=180n
M4610 nw635 t1669 0 0 nch w=1u l=180n
Cnw635 nw635 0 2f
CT1671 t1671 0 0.1f
M4611 t1671 nw574 0 0 nch w=1u l=180n
M4612 t1671 nw540 0 0 nch w=1u l=180n
CT1672 t1672 0 0.1f
M4613 t1672 nw574 vdd vdd pch w=2u l=180n
M4614 t1671 nw540 t1672 vdd pch w=2u l=180n
M4615 nw636 t1671 vdd vdd pch w=2u l=180n
M4616 nw636 t1671 0 0 nch w=1u l=180n
Cnw636 nw636 0 2f
CT1673 t1673 0 0.1f
CT1674 t1674 0 0.1f
CT1675 t1675 0 0.1f
M4617 t1673 nw575 vdd vdd pch w=2u l=180n
M4618 t1673 nw541 vdd vdd pch w=2u l=180n
CT1676 t1676 0 0.1f
M4619 t1673 nw575 t1676 0 nch w=1u l=180n
M4620 t1676 nw541 0 0 nch w=1u l=180n
M4621 t1674 nw575 vdd vdd pch w=2u l=180n
M4622 t1674 t1673 vdd vdd pch w=2u l=180n
CT1677 t1677 0 0.1f
M4623 t1674 nw575 t1677 0 nch w=1u l=180n
M4624 t1677 t1673 0 0 nch w=1u l=180n
M4625 t1675 nw541 vdd vdd pch w=2u l=180n
M4626 t1675 t1673 vdd vdd pch w=2u l=180n
CT1678 t1678 0 0.1f
M4627 t1675 nw541 t1678 0 nch w=1u l=180n
M4628 t1678 t1673 0 0 nch w=1u l=180n
M4629 nw637 t1674 vdd vdd pch w=2u l=180n
M4630 nw637 t1675 vdd vdd pch w=2u l=180n
CT1679 t1679 0 0.1f
M4631 nw637 t1674 t1679 0 nch w=1u l=180n
M4632 t1679 t1675 0 0 nch w=1u l=180n
Cnw637 nw637 0 2f
M4633 nw638 nw576 vdd vdd pch w=2u l=180n
M4634 nw638 nw542 vdd vdd pch w=2u l=180n
CT1680 t1680 0 0.1f
M4635 nw638 nw576 t1680 0 nch w=1u l=180n
M4636 t1680 nw542 0 0 nch w=1u l=180n
Cnw638 nw638 0 2f
M4637 nw639 nw577 0 0 nch w=1u l=180n
M4638 nw639 nw543 0 0 nch w=1u l=180n
CT1681 t1681 0 0.1f
M4639 t1681 nw577 vdd vdd pch w=2u l=180n
M4640 nw639 nw543 t1681 vdd pch w=2u l=180n
Cnw639 nw639 0 2f
CT1682 t1682 0 0.1f
M4641 t1682 nw578 vdd vdd pch w=2u l=180n
M4642 t1682 nw544 vdd vdd pch w=2u l=180n
CT1683 t1683 0 0.1f
M4643 t1682 nw578 t1683 0 nch w=1u l=180n
M4644 t1683 nw544 0 0 nch w=1u l=180n
M4645 nw640 t1682 vdd vdd pch w=2u l=180n
M4646 nw640 t1682 0 0 nch w=1u l=180n
Cnw640 nw640 0 2f
CT1684 t1684 0 0.1f
M4647 t1684 nw579 0 0 nch w=1u l=180n
M4648 t1684 nw545 0 0 nch w=1u l=180n
CT1685 t1685 0 0.1f
M4649 t1685 nw579 vdd vdd pch w=2u l=180n
M4650 t1684 nw545 t1685 vdd pch w=2u l=180n
M4651 nw641 t1684 vdd vdd pch w=2u l=180n
M4652 nw641 t1684 0 0 nch w=1u l=180n
Cnw641 nw641 0 2f
CT1686 t1686 0 0.1f
CT1687 t1687 0 0.1f
CT1688 t1688 0 0.1f
M4653 t1686 nw580 vdd vdd pch w=2u l=180n
M4654 t1686 nw546 vdd vdd pch w=2u l=180n
CT1689 t1689 0 0.1f
M4655 t1686 nw580 t1689 0 nch w=1u l=180n
M4656 t1689 nw546 0 0 nch w=1u l=180n
M4657 t1687 nw580 vdd vdd pch w=2u l=180n
M4658 t1687 t1686 vdd vdd pch w=2u l=180n
CT1690 t1690 0 0.1f
M4659 t1687 nw580 t1690 0 nch w=1u l=180n
M4660 t1690 t1686 0 0 nch w=1u l=180n
M4661 t1688 nw546 vdd vdd pch w=2u l=180n
M4662 t1688 t1686 vdd vdd pch w=2u l=180n
CT1691 t1691 0 0.1f
M4663 t1688 nw546 t1691 0 nch w=1u l=180n
M4664 t1691 t1686 0 0 nch w=1u l=180n
M4665 nw642 t1687 vdd vdd pch w=2u l=180n
M4666 nw642 t1688 vdd vdd pch w=2u l=180n
CT1692 t1692 0 0.1f
M4667 nw642 t1687 t1692 0 nch w=1u l=180n
M4668 t1692 t1688 0 0 nch w=1u l=180n
Cnw642 nw642 0 2f
M4669 nw643 nw581 vdd vdd pch w=2u l=180n
M4670 nw643 nw547 vdd vdd pch w=2u l=180n
CT1693 t1693 0 0.1f
M4671 nw643 nw581 t1693 0 nch w=1u l=180n
M4672 t1693 nw547 0 0 nch w=1u l=180n
Cnw643 nw643 0 2f
M4673 nw644 nw582 0 0 nch w=1u l=180n
M4674 nw644 nw548 0 0 nch w=1u l=180n
CT1694 t1694 0 0.1f
M4675 t1694 nw582 vdd vdd pch w=2u l=180n
M4676 nw644 nw548 t1694 vdd pch w=2u l=180n
Cnw644 nw644 0 2f
CT1695 t1695 0 0.1f
M4677 t1695 nw583 vdd vdd pch w=2u l=180n
M4678 t1695 nw549 vdd vdd pch w=2u l=180n
CT1696 t1696 0 0.1f
M4679 t1695 nw583 t1696 0 nch w=1u l=180n
M4680 t1696 nw549 0 0 nch w=1u l=180n
M4681 nw645 t1695 vdd vdd pch w=2u l=180n
M4682 nw645 t1695 0 0 nch w=1u l=180n
Cnw645 nw645 0 2f
CT1697 t1697 0 0.1f
M4683 t1697 nw584 0 0 nch w=1u l=180n
M4684 t1697 nw550 0 0 nch w=1u l=180n
CT1698 t1698 0 0.1f
M4685 t1698 nw584 vdd vdd pch w=2u l=180n
M4686 t1697 nw550 t1698 vdd pch w=2u l=180n
M4687 nw646 t1697 vdd vdd pch w=2u l=180n
M4688 nw646 t1697 0 0 nch w=1u l=180n
Cnw646 nw646 0 2f
CT1699 t1699 0 0.1f
CT1700 t1700 0 0.1f
CT1701 t1701 0 0.1f
M4689 t1699 nw585 vdd vdd pch w=2u l=180n
M4690 t1699 nw551 vdd vdd pch w=2u l=180n
CT1702 t1702 0 0.1f
M4691 t1699 nw585 t1702 0 nch w=1u l=180n
M4692 t1702 nw551 0 0 nch w=1u l=180n
M4693 t1700 nw585 vdd vdd pch w=2u l=180n
M4694 t1700 t1699 vdd vdd pch w=2u l=180n
CT1703 t1703 0 0.1f
M4695 t1700 nw585 t1703 0 nch w=1u l=180n
M4696 t1703 t1699 0 0 nch w=1u l=180n
M4697 t1701 nw551 vdd vdd pch w=2u l=180n
M4698 t1701 t1699 vdd vdd pch w=2u l=180n
CT1704 t1704 0 0.1f
M4699 t1701 nw551 t1704 0 nch w=1u l=180n
M4700 t1704 t1699 0 0 nch w=1u l=180n
M4701 nw647 t1700 vdd vdd pch w=2u l=180n
M4702 nw647 t1701 vdd vdd pch w=2u l=180n
CT1705 t1705 0 0.1f
M4703 nw647 t1700 t1705 0 nch w=1u l=180n
M4704 t1705 t1701 0 0 nch w=1u l=180n
Cnw647 nw647 0 2f
M4705 nw648 nw586 vdd vdd pch w=2u l=180n
M4706 nw648 nw552 vdd vdd pch w=2u l=180n
CT1706 t1706 0 0.1f
M4707 nw648 nw586 t1706 0 nch w=1u l=180n
M4708 t1706 nw552 0 0 nch w=1u l=180n
Cnw648 nw648 0 2f
M4709 nw649 nw587 0 0 nch w=1u l=180n
M4710 nw649 nw553 0 0 nch w=1u l=180n
CT1707 t1707 0 0.1f
M4711 t1707 nw587 vdd vdd pch w=2u l=180n
M4712 nw649 nw553 t1707 vdd pch w=2u l=180n
Cnw649 nw649 0 2f
CT1708 t1708 0 0.1f
M4713 t1708 nw588 vdd vdd pch w=2u l=180n
M4714 t1708 nw554 vdd vdd pch w=2u l=180n
CT1709 t1709 0 0.1f
M4715 t1708 nw588 t1709 0 nch w=1u l=180n
M4716 t1709 nw554 0 0 nch w=1u l=180n
M4717 nw650 t1708 vdd vdd pch w=2u l=180n
M4718 nw650 t1708 0 0 nch w=1u l=180n
Cnw650 nw650 0 2f
CT1710 t1710 0 0.1f
M4719 t1710 nw589 0 0 nch w=1u l=180n
M4720 t1710 nw555 0 0 nch w=1u l=180n
CT1711 t1711 0 0.1f
M4721 t1711 nw589 vdd vdd pch w=2u l=180n
M4722 t1710 nw555 t1711 vdd pch w=2u l=180n
M4723 nw651 t1710 vdd vdd pch w=2u l=180n
M4724 nw651 t1710 0 0 nch w=1u l=180n
Cnw651 nw651 0 2f
CT1712 t1712 0 0.1f
CT1713 t1713 0 0.1f
CT1714 t1714 0 0.1f
M4725 t1712 nw590 vdd vdd pch w=2u l=180n
M4726 t1712 nw556 vdd vdd pch w=2u l=180n
CT1715 t1715 0 0.1f
M4727 t1712 nw590 t1715 0 nch w=1u l=180n
M4728 t1715 nw556 0 0 nch w=1u l=180n
M4729 t1713 nw590 vdd vdd pch w=2u l=180n
M4730 t1713 t1712 vdd vdd pch w=2u l=180n
CT1716 t1716 0 0.1f
M4731 t1713 nw590 t1716 0 nch w=1u l=180n
M4732 t1716 t1712 0 0 nch w=1u l=180n
M4733 t1714 nw556 vdd vdd pch w=2u l=180n
M4734 t1714 t1712 vdd vdd pch w=2u l=180n
CT1717 t1717 0 0.1f
M4735 t1714 nw556 t1717 0 nch w=1u l=180n
M4736 t1717 t1712 0 0 nch w=1u l=180n
M4737 nw652 t1713 vdd vdd pch w=2u l=180n
M4738 nw652 t1714 vdd vdd pch w=2u l=180n
CT1718 t1718 0 0.1f
M4739 nw652 t1713 t1718 0 nch w=1u l=180n
M4740 t1718 t1714 0 0 nch w=1u l=180n
Cnw652 nw652 0 2f
M4741 nw653 nw591 vdd vdd pch w=2u l=180n
M4742 nw653 nw557 vdd vdd pch w=2u l=180n
CT1719 t1719 0 0.1f
M4743 nw653 nw591 t1719 0 nch w=1u l=180n
M4744 t1719 nw557 0 0 nch w=1u l=180n
Cnw653 nw653 0 2f
M4745 nw654 nw592 0 0 nch w=1u l=180n
M4746 nw654 nw558 0 0 nch w=1u l=180n
CT1720 t1720 0 0.1f
M4747 t1720 nw592 vdd vdd pch w=2u l=180n
M4748 nw654 nw558 t1720 vdd pch w=2u l=180n
Cnw654 nw654 0 2f
CT1721 t1721 0 0.1f
M4749 t1721 nw593 vdd vdd pch w=2u l=180n
M4750 t1721 nw559 vdd vdd pch w=2u l=180n
CT1722 t1722 0 0.1f
M4751 t1721 nw593 t1722 0 nch w=1u l=180n
M4752 t1722 nw559 0 0 nch w=1u l=180n
M4753 nw655 t1721 vdd vdd pch w=2u l=180n
M4754 nw655 t1721 0 0 nch w=1u l=180n
Cnw655 nw655 0 2f
CT1723 t1723 0 0.1f
M4755 t1723 nw594 0 0 nch w=1u l=180n
M4756 t1723 nw560 0 0 nch w=1u l=180n
CT1724 t1724 0 0.1f
M4757 t1724 nw594 vdd vdd pch w=2u l=180n
M4758 t1723 nw560 t1724 vdd pch w=2u l=180n
M4759 nw656 t1723 vdd vdd pch w=2u l=180n
M4760 nw656 t1723 0 0 nch w=1u l=180n
Cnw656 nw656 0 2f
CT1725 t1725 0 0.1f
CT1726 t1726 0 0.1f
CT1727 t1727 0 0.1f
M4761 t1725 nw595 vdd vdd pch w=2u l=180n
M4762 t1725 nw561 vdd vdd pch w=2u l=180n
CT1728 t1728 0 0.1f
M4763 t1725 nw595 t1728 0 nch w=1u l=180n
M4764 t1728 nw561 0 0 nch w=1u l=180n
M4765 t1726 nw595 vdd vdd pch w=2u l=180n
M4766 t1726 t1725 vdd vdd pch w=2u l=180n
CT1729 t1729 0 0.1f
M4767 t1726 nw595 t1729 0 nch w=1u l=180n
M4768 t1729 t1725 0 0 nch w=1u l=180n
M4769 t1727 nw561 vdd vdd pch w=2u l=180n
M4770 t1727 t1725 vdd vdd pch w=2u l=180n
CT1730 t1730 0 0.1f
M4771 t1727 nw561 t1730 0 nch w=1u l=180n
M4772 t1730 t1725 0 0 nch w=1u l=180n
M4773 nw657 t1726 vdd vdd pch w=2u l=180n
M4774 nw657 t1727 vdd vdd pch w=2u l=180n
CT1731 t1731 0 0.1f
M4775 nw657 t1726 t1731 0 nch w=1u l=180n
M4776 t1731 t1727 0 0 nch w=1u l=180n
Cnw657 nw657 0 2f
M4777 nw658 nw596 vdd vdd pch w=2u l=180n
M4778 nw658 nw562 vdd vdd pch w=2u l=180n
CT1732 t1732 0 0.1f
M4779 nw658 nw596 t1732 0 nch w=1u l=180n
M4780 t1732 nw562 0 0 nch w=1u l=180n
Cnw658 nw658 0 2f
M4781 nw659 nw597 0 0 nch w=1u l=180n
M4782 nw659 nw563 0 0 nch w=1u l=180n
CT1733 t1733 0 0.1f
M4783 t1733 nw597 vdd vdd pch w=2u l=180n
M4784 nw659 nw563 t1733 vdd pch w=2u l=180n
Cnw659 nw659 0 2f
CT1734 t1734 0 0.1f
M4785 t1734 nw598 vdd vdd pch w=2u l=180n
M4786 t1734 nw564 vdd vdd pch w=2u l=180n
CT1735 t1735 0 0.1f
M4787 t1734 nw598 t1735 0 nch w=1u l=180n
M4788 t1735 nw564 0 0 nch w=1u l=180n
M4789 nw660 t1734 vdd vdd pch w=2u l=180n
M4790 nw660 t1734 0 0 nch w=1u l=180n
Cnw660 nw660 0 2f
CT1736 t1736 0 0.1f
M4791 t1736 nw599 0 0 nch w=1u l=180n
M4792 t1736 nw565 0 0 nch w=1u l=180n
CT1737 t1737 0 0.1f
M4793 t1737 nw599 vdd vdd pch w=2u l=180n
M4794 t1736 nw565 t1737 vdd pch w=2u l=180n
M4795 nw661 t1736 vdd vdd pch w=2u l=180n
M4796 nw661 t1736 0 0 nch w=1u l=180n
Cnw661 nw661 0 2f
CT1738 t1738 0 0.1f
CT1739 t1739 0 0.1f
CT1740 t1740 0 0.1f
M4797 t1738 nw600 vdd vdd pch w=2u l=180n
M4798 t1738 nw566 vdd vdd pch w=2u l=180n
CT1741 t1741 0 0.1f
M4799 t1738 nw600 t1741 0 nch w=1u l=180n
M4800 t1741 nw566 0 0 nch w=1u l=180n
M4801 t1739 nw600 vdd vdd pch w=2u l=180n
M4802 t1739 t1738 vdd vdd pch w=2u l=180n
CT1742 t1742 0 0.1f
M4803 t1739 nw600 t1742 0 nch w=1u l=180n
M4804 t1742 t1738 0 0 nch w=1u l=180n
M4805 t1740 nw566 vdd vdd pch w=2u l=180n
M4806 t1740 t1738 vdd vdd pch w=2u l=180n
CT1743 t1743 0 0.1f
M4807 t1740 nw566 t1743 0 nch w=1u l=180n
M4808 t1743 t1738 0 0 nch w=1u l=180n
M4809 nw662 t1739 vdd vdd pch w=2u l=180n
M4810 nw662 t1740 vdd vdd pch w=2u l=180n
CT1744 t1744 0 0.1f
M4811 nw662 t1739 t1744 0 nch w=1u l=180n
M4812 t1744 t1740 0 0 nch w=1u l=180n
Cnw662 nw662 0 2f
CT1745 t1745 0 0.1f
M4813 t1745 nw662 vdd vdd pch w=2u l=180n
M4814 t1745 nw662 0 0 nch w=1u l=180n
M4815 no0 t1745 vdd vdd pch w=2u l=180n
M4816 no0 t1745 0 0 nch w=1u l=180n
Cno0 no0 0 2f
CT1746 t1746 0 0.1f
M4817 t1746 nw661 vdd vdd pch w=2u l=180n
M4818 t1746 nw661 0 0 nch w=1u l=180n
M4819 no1 t1746 vdd vdd pch w=2u l=180n
M4820 no1 t1746 0 0 nch w=1u l=180n
Cno1 no1 0 2f
CT1747 t1747 0 0.1f
M4821 t1747 nw660 vdd vdd pch w=2u l=180n
M4822 t1747 nw660 0 0 nch w=1u l=180n
M4823 no2 t1747 vdd vdd pch w=2u l=180n
M4824 no2 t1747 0 0 nch w=1u l=180n
Cno2 no2 0 2f
CT1748 t1748 0 0.1f
M4825 t1748 nw659 vdd vdd pch w=2u l=180n
M4826 t1748 nw659 0 0 nch w=1u l=180n
M4827 no3 t1748 vdd vdd pch w=2u l=180n
M4828 no3 t1748 0 0 nch w=1u l=180n
Cno3 no3 0 2f
CT1749 t1749 0 0.1f
M4829 t1749 nw658 vdd vdd pch w=2u l=180n
M4830 t1749 nw658 0 0 nch w=1u l=180n
M4831 no4 t1749 vdd vdd pch w=2u l=180n
M4832 no4 t1749 0 0 nch w=1u l=180n
Cno4 no4 0 2f
CT1750 t1750 0 0.1f
M4833 t1750 nw657 vdd vdd pch w=2u l=180n
M4834 t1750 nw657 0 0 nch w=1u l=180n
M4835 no5 t1750 vdd vdd pch w=2u l=180n
M4836 no5 t1750 0 0 nch w=1u l=180n
Cno5 no5 0 2f
CT1751 t1751 0 0.1f
M4837 t1751 nw656 vdd vdd pch w=2u l=180n
M4838 t1751 nw656 0 0 nch w=1u l=180n
M4839 no6 t1751 vdd vdd pch w=2u l=180n
M4840 no6 t1751 0 0 nch w=1u l=180n
Cno6 no6 0 2f
CT1752 t1752 0 0.1f
M4841 t1752 nw655 vdd vdd pch w=2u l=180n
M4842 t1752 nw655 0 0 nch w=1u l=180n
M4843 no7 t1752 vdd vdd pch w=2u l=180n
M4844 no7 t1752 0 0 nch w=1u l=180n
Cno7 no7 0 2f
.model nch NMOS (vto=0.45 kp=200u lambda=0.05)
.model pch PMOS (vto=-0.45 kp=100u lambda=0.05)
* outputs: nw1 nw3 nw5 nw7 nw9 nw11 no0 no1 no2 no3 no4 no5 no6 no7
.end
